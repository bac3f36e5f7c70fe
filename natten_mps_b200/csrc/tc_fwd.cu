// Fused neighbourhood-attention forward on tcgen05 tensor cores (sm_100a).
//
// One CTA handles a box of 128 queries of one (batch, head): the union of their
// neighbourhoods is a box of keys, walked in chunks of 128 keys.  Per chunk
//   S = Q K^T      tcgen05.mma, operands staged by TMA (128-byte swizzle), accumulator in TMEM
//   P = exp2(S*scale*log2e - max)   softmax warps, one query row per thread, read S from TMEM,
//                                   apply the window mask, write P (16-bit) back to TMEM
//   O_c = P V      tcgen05.mma with A = P from TMEM, B = V tile read MN-major
// and the threads fold O_c into register accumulators with the usual running-max
// rescale.  One extra warp issues every TMA load and MMA.  Geometry (rank, window,
// dilation, causal axes, per-sample extents) is runtime data; masks are built per
// 32-column piece from per-row box ranges.  Dilation is handled as independent
// sub-grids, loaded through the tensor map's element strides.
//
// TMEM columns per CTA (256):  S [0,128)  P [128,192)  O [192,256).
// Shared memory per CTA: Q 16 KB + 3 stages x (K 16 KB + V 16 KB) = 112 KB -> two CTAs per SM.
#include "tc_kernels.cuh"

#include "tc_plan.cuh"

#include <type_traits>

namespace natten {

using namespace tc;
using namespace tcplan;

__device__ int g_tc_status = 0;

static long long* g_trace = nullptr;
void tc_set_trace(void* p) { g_trace = reinterpret_cast<long long*>(p); }

namespace tcplan {
long long* trace_ptr() { return g_trace; }
int* status_ptr()
{
    int* p = nullptr;
    cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_tc_status);
    return p;
}
} // namespace tcplan

namespace {

constexpr int kThreads = 320;            // 8 softmax warps + MMA warp + TMA warp
constexpr uint32_t kColS = 0, kColP = 128;      // S: 128 columns, P: 64; O follows (64 or 128 columns)

// Shared-memory map (dynamic, base must be 1024-byte aligned).
template <int DH>
struct SmemMap {
    static constexpr int kHalves = DH / 64;                       // 64-channel blocks (one swizzle row each)
    static constexpr int kKStages = 3;                            // K is released right after Q K^T, so it runs further ahead
    static constexpr int kVStages = 2;                            // V is released after P V
    static constexpr int kQBufs = 2;                              // next tile's queries load during this tile
    static constexpr int kHalf = kTileRows * 128;                 // bytes of one [128 x 64] 16-bit block
    static constexpr int kTile = kHalf * kHalves;                 // bytes of one [128 x DH] 16-bit tile
    static constexpr int kQ = 0;
    static constexpr int kK = kQ + kQBufs * kTile;
    static constexpr int kV = kK + kKStages * kTile;
    static constexpr int kBar = kV + kVStages * kTile;
    // barriers (q, k, v full/empty per buffer, s, sr, sp, o), abort flag, TMEM slot: 192 bytes,
    // then 512 bytes for the two column halves to exchange their row maxima.
    // Two CTAs share an SM only while kTotal + 1 KB (reserved per CTA) <= 114 KB.
    static constexpr int kTotal = kBar + 192 + 512;
    static_assert(DH != 64 || 2 * (kTotal + 1024) <= 233472, "two CTAs per SM must fit");
    static constexpr uint32_t kTmemCols = DH == 64 ? 256 : 512;
    static constexpr uint32_t kColO = DH == 64 ? 192 : 256;
};

__device__ __forceinline__ int tc_window_start(int p, int L, int K) { return window_start(p, L, K, 1); }

// Geometry of one work item: a tile of 128 queries of one (batch, head).
struct FwdTile {
    int b, h, hk;
    int rg[3], origin[3], Lp[3], lo[3], nc[3];
    int nnb, nch;            // chunks of the neighbourhood box / including the additional tokens
    bool active;
};

__device__ __forceinline__ void fwd_tile_setup(const TcParams& P, unsigned work, FwdTile& T)
{
    const unsigned hb = work / P.per_head;
    const unsigned bx = work - hb * P.per_head;
    T.b = (int)(hb / (unsigned)P.Hq);
    T.h = (int)(hb - (unsigned)T.b * (unsigned)P.Hq);
    T.hk = T.h / P.group;
    T.active = cta_geometry(P, bx, T.b, T.rg, T.origin, T.Lp);
    T.nnb = 1;
    if (T.active) {
#pragma unroll
        for (int a = 0; a < 3; ++a) {
            const int last = T.origin[a] + P.tile[a] - 1 < T.Lp[a] - 1 ? T.origin[a] + P.tile[a] - 1 : T.Lp[a] - 1;
            T.lo[a] = P.causal[a] ? T.origin[a] - (P.K[a] - 1) : tc_window_start(T.origin[a], T.Lp[a], P.K[a]);
            const int hi = P.causal[a] ? last : tc_window_start(last, T.Lp[a], P.K[a]) + P.K[a] - 1;
            T.nc[a] = chunks_along(P, a, hi - T.lo[a] + 1);   // chunks this tile really needs
            T.nnb *= T.nc[a];
        }
    }
    T.nch = T.nnb + ((P.n_extra + kChunk - 1) >> 7);          // then the additional tokens, 128 per chunk
}

// Persistent kernel: every CTA walks the work items blockIdx.x, blockIdx.x + gridDim.x, ...
// Warps 0-7 softmax, warp 8 issues the MMAs, warp 9 issues the TMA loads (it runs ahead across
// tiles, bounded by the K/V stages and the single Q buffer).  Barrier phases run on across tiles.
// kInner: innermost chunk extent when it is 16 or 32 (separable row / column masks),
// 0 = any geometry (per-column validity words from piece_word).
template <int DH, bool BF16, int kInner>
__global__ void __launch_bounds__(kThreads, (DH == 64 ? 2 : 1))
tc_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
              const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmEK,
              const __grid_constant__ CUtensorMap tmEV, const __grid_constant__ TcParams P,
              uint16_t* __restrict__ out, float* __restrict__ lse)
{
    using SM = SmemMap<DH>;
    constexpr int kKStages = SM::kKStages, kVStages = SM::kVStages;
    constexpr int CH = DH / 2;                 // output channels per softmax thread
    constexpr uint32_t kColO = SM::kColO, kTmemCols = SM::kTmemCols;
    extern __shared__ __align__(1024) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int quad = warp & 3, team = (warp >> 2) & 1;        // softmax warps: TMEM lane quadrant, column half
    const int prior_abort = *reinterpret_cast<volatile int*>(P.status);

    const uint32_t sbase = smem_u32(smem);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + SM::kBar + 176);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + SM::kBar + 184);
    uint16_t* xmax = reinterpret_cast<uint16_t*>(smem + SM::kBar + 192);      // [2 halves][128] row maxima (bf16 bits)
    const uint32_t bar_q_full = sbase + SM::kBar + 0;       // [2]
    const uint32_t bar_q_empty = sbase + SM::kBar + 16;     // [2]
    const uint32_t bar_k_full = sbase + SM::kBar + 32;      // [kKStages]
    const uint32_t bar_k_empty = sbase + SM::kBar + 56;     // [kKStages]
    const uint32_t bar_v_full = sbase + SM::kBar + 80;      // [kVStages]
    const uint32_t bar_v_empty = sbase + SM::kBar + 96;     // [kVStages]
    const uint32_t bar_s = sbase + SM::kBar + 112;
    const uint32_t bar_sp = sbase + SM::kBar + 120;
    const uint32_t bar_o = sbase + SM::kBar + 128;
    const uint32_t bar_sr = sbase + SM::kBar + 136;         // every softmax thread holds S(c) in registers

    if (warp == 8) {
        if (lane == 0) {
            // swizzled tiles need a 1024-byte aligned base; once any CTA has given up, the rest bail out
            *abort_flag = ((sbase & 1023u) || prior_abort) ? 1 : 0;
            for (int i = 0; i < 2; ++i) { mbar_init(bar_q_full + 8 * i, 1); mbar_init(bar_q_empty + 8 * i, 1); }
            for (int s = 0; s < kKStages; ++s) { mbar_init(bar_k_full + 8 * s, 1); mbar_init(bar_k_empty + 8 * s, 1); }
            for (int s = 0; s < kVStages; ++s) { mbar_init(bar_v_full + 8 * s, 1); mbar_init(bar_v_empty + 8 * s, 1); }
            mbar_init(bar_s, 1);
            mbar_init(bar_sp, 256);
            mbar_init(bar_o, 1);
            mbar_init(bar_sr, 256);
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
    // debug clock stamps of the first work item of CTA 5: forward uses entries [256, 384)
    long long* tr = (P.trace && blockIdx.x == 5) ? P.trace + 256 : nullptr;
    int tn = 0;
    auto stamp = [&](int base) { if (tr && tn < 60) tr[base + tn++] = clock64(); };
    const long long t_begin = clock64();

    if (warp == 9) {
        // =====================================================================
        // TMA producers: lane 0 streams Q (once per tile) and the K chunks, lane 1 streams the V
        // chunks.  Each runs ahead across tiles as far as its own buffers allow.
        // =====================================================================
        if (lane < 2 && !*abort_flag) {
            const bool is_k = lane == 0;
            const CUtensorMap* map = is_k ? &tmK : &tmV;
            const CUtensorMap* emap = is_k ? &tmEK : &tmEV;
            const int nstage = is_k ? kKStages : kVStages;
            const uint32_t bar_full = is_k ? bar_k_full : bar_v_full;
            const uint32_t bar_empty = is_k ? bar_k_empty : bar_v_empty;
            const uint32_t sdst = sbase + (is_k ? SM::kK : SM::kV);
            unsigned gl = 0, tq = 0;                      // loads / tiles issued so far by this stream
            bool ok = true;
            for (unsigned work = blockIdx.x; work < P.work_q && ok; work += gridDim.x) {
                FwdTile T;
                fwd_tile_setup(P, work, T);
                if (!T.active) continue;
                if (is_k) {
                    const unsigned qb = tq & 1;          // Q buffer of this tile
                    if (tq >= 2) ok = mbar_wait(bar_q_empty + 8 * qb, ((tq >> 1) - 1) & 1, abort_flag);   // its last user's QK MMAs done
                    if (!ok) break;
                    mbar_expect_tx(bar_q_full + 8 * qb, SM::kTile);
#pragma unroll
                    for (int hf = 0; hf < SM::kHalves; ++hf)
                        tma_load_5d(sbase + SM::kQ + qb * SM::kTile + hf * SM::kHalf, &tmQ, bar_q_full + 8 * qb, T.h * DH + 64 * hf,
                                    T.rg[2] + P.dil[2] * T.origin[2], T.rg[1] + P.dil[1] * T.origin[1],
                                    T.rg[0] + P.dil[0] * T.origin[0], T.b);
                }
                ++tq;
                int ld[3] = {0, 0, 0};
                for (int c = 0; c < T.nch && ok; ++c, ++gl) {
                    const unsigned s = gl % nstage;
                    if (gl >= (unsigned)nstage) ok = mbar_wait(bar_empty + 8 * s, ((gl / nstage) - 1) & 1, abort_flag);
                    if (!ok) break;
                    const uint32_t bar = bar_full + 8 * s;
                    mbar_expect_tx(bar, SM::kTile);
                    if (c < T.nnb) {
                        int X[3];
#pragma unroll
                        for (int a = 0; a < 3; ++a) X[a] = T.rg[a] + P.dil[a] * (T.lo[a] + ld[a] * P.cb[a]);
#pragma unroll
                        for (int hf = 0; hf < SM::kHalves; ++hf)
                            tma_load_5d(sdst + s * SM::kTile + hf * SM::kHalf, map, bar, T.hk * DH + 64 * hf, X[2], X[1], X[0], T.b);
                        if (++ld[2] == T.nc[2]) { ld[2] = 0; if (++ld[1] == T.nc[1]) { ld[1] = 0; ++ld[0]; } }
                    } else {                             // additional tokens (rows past n_extra are zero-filled)
                        const int e0 = (c - T.nnb) * kChunk;
#pragma unroll
                        for (int hf = 0; hf < SM::kHalves; ++hf)
                            tma_load_5d(sdst + s * SM::kTile + hf * SM::kHalf, emap, bar, T.hk * DH + 64 * hf, e0, 0, 0, T.b);
                    }
                }
            }
        }
    } else if (warp == 8) {
        // =====================================================================
        // MMA issue (one thread)
        // =====================================================================
        if (lane == 0 && !*abort_flag) {
            constexpr uint32_t idesc_qk = instr_desc(BF16 ? 1 : 0, kChunk, 0, 0);
            constexpr uint32_t idesc_pv = instr_desc(BF16 ? 1 : 0, DH, 0, 1);
            auto issue_qk = [&](unsigned g, uint64_t dq0) {
                const uint64_t dk0 = smem_desc(sbase + SM::kK + (g % kKStages) * SM::kTile, 16, 1024);
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < DH / 16; ++ks) {       // 32 bytes per k-step inside a 64-channel block
                    const uint32_t off = ((ks / 4) * SM::kHalf + (ks % 4) * 32) >> 4;
                    mma_ss(tmem + kColS, dq0 + off, dk0 + off, idesc_qk, ks > 0);
                }
                mma_commit(bar_s);
                mma_commit(bar_k_empty + 8 * (g % kKStages));        // the K stage can be reloaded
            };
            auto issue_pv = [&](unsigned g, bool accumulate) {
                // V read MN-major: 16 key rows per k-step, the second 64-channel block sits kHalf bytes further.
                // O stays in TMEM for the whole tile: every chunk after the first adds to it.
                const uint64_t dv0 = smem_desc(sbase + SM::kV + (g % kVStages) * SM::kTile, SM::kHalf, 1024);
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < kChunk / 16; ++ks)
                    mma_ts(tmem + kColO, tmem + kColP + 8 * ks, dv0 + 128 * ks, idesc_pv, accumulate || ks > 0);
                mma_commit(bar_o);
                mma_commit(bar_v_empty + 8 * (g % kVStages));        // the V stage can be reloaded
            };
            // next work item of this CTA that has anything to attend
            auto next_active = [&](unsigned w, FwdTile& X) {
                for (; w < P.work_q; w += gridDim.x) {
                    fwd_tile_setup(P, w, X);
                    if (X.active) break;
                }
                return w;
            };
            unsigned gc = 0, tq = 0;                      // chunks / tiles processed so far
            bool ok = true;
            // first scores of a tile: its queries and its first keys have landed
            auto first_qk = [&](const FwdTile& X, unsigned t, unsigned g) {
                const unsigned qb = t & 1;
                ok = mbar_wait(bar_q_full + 8 * qb, (t >> 1) & 1, abort_flag) &&
                     mbar_wait(bar_k_full + 8 * (g % kKStages), (g / kKStages) & 1, abort_flag);
                if (!ok) return;
                issue_qk(g, smem_desc(sbase + SM::kQ + qb * SM::kTile, 16, 1024));
                if (X.nch == 1) mma_commit(bar_q_empty + 8 * qb);
            };
            FwdTile T, Tn;
            unsigned work = next_active(blockIdx.x, T);
            if (work < P.work_q) first_qk(T, 0, 0);
            while (work < P.work_q && ok) {
                stamp(0);
                const unsigned qb = tq & 1;
                const uint64_t dq0 = smem_desc(sbase + SM::kQ + qb * SM::kTile, 16, 1024);
                unsigned wnext = P.work_q;
                for (int c = 0; c < T.nch && ok; ++c, ++gc) {
                    const bool last = c + 1 == T.nch;
                    if (last) wnext = next_active(work + gridDim.x, Tn);
                    // S(c) sits in the threads' registers: the next scores may overwrite it while they work
                    ok = mbar_wait(bar_sr, gc & 1, abort_flag);
                    if (!ok) break;
                    stamp(0);
                    if (!last) {
                        ok = mbar_wait(bar_k_full + 8 * ((gc + 1) % kKStages), ((gc + 1) / kKStages) & 1, abort_flag);
                        if (!ok) break;
                        issue_qk(gc + 1, dq0);
                        if (c + 2 == T.nch) mma_commit(bar_q_empty + 8 * qb);   // last QK of the tile: its Q buffer is free after it
                    } else if (wnext < P.work_q) {
                        first_qk(Tn, tq + 1, gc + 1);
                        if (!ok) break;
                    }
                    ok = mbar_wait(bar_sp, gc & 1, abort_flag);          // P(c) stored
                    if (!ok) break;
                    stamp(0);
                    ok = mbar_wait(bar_v_full + 8 * (gc % kVStages), (gc / kVStages) & 1, abort_flag);
                    if (!ok) break;
                    issue_pv(gc, c > 0);
                    stamp(0);
                }
                T = Tn;
                work = wnext;
                ++tq;
            }
        }
    } else {
        // =====================================================================
        // softmax warps: thread = (query row, 64-column half of the chunk, CH output channels)
        // =====================================================================
        const uint32_t trow = tmem + (static_cast<uint32_t>(quad * 32) << 16);
        const int row = quad * 32 + lane;
        bool ok = true;
        unsigned gc = 0;                                 // chunks processed so far (all tiles)
        for (unsigned work = blockIdx.x; work < P.work_q; work += gridDim.x) {
            FwdTile T;
            fwd_tile_setup(P, work, T);
            // ---- this thread's query row ----
            int f[3] = {0, 0, 0}, e[3] = {0, 0, 0};
            bool valid_q = true, in_tensor = true;
            long long pflat = 0;
            {
                int qi[3];
                row_offsets(P, row, qi);
#pragma unroll
                for (int a = 0; a < 3; ++a) {
                    const int qa = T.origin[a] + qi[a];
                    const int pa = T.rg[a] + P.dil[a] * qa;
                    if (qa >= T.Lp[a]) valid_q = false;
                    if (pa >= P.L[a]) in_tensor = false;
                    pflat = pflat * P.L[a] + pa;
                    if (T.active) {
                        const int first = P.causal[a] ? qa - (P.K[a] - 1) : tc_window_start(qa, T.Lp[a], P.K[a]);
                        f[a] = (first > 0 ? first : 0) - T.lo[a];
                        e[a] = (first + P.K[a] < T.Lp[a] ? first + P.K[a] : T.Lp[a]) - T.lo[a];
                    }
                }
                if (!valid_q) { e[0] = f[0]; e[1] = f[1]; e[2] = f[2]; }
            }
            const long long out_row = (((long long)T.b * P.ltot + pflat) * P.Hq + T.h);
            if (!T.active) {                     // nothing to attend: padding rows are zero
                if (in_tensor) {
                    uint4* o4 = reinterpret_cast<uint4*>(out + out_row * DH + team * CH);
#pragma unroll
                    for (int i = 0; i < CH / 8; ++i) o4[i] = make_uint4(0, 0, 0, 0);
                    if (team == 0) lse[out_row] = 0.f;
                }
                continue;
            }

            // O accumulates in TMEM over the tile's chunks.  m is the stabiliser the stored
            // probabilities use; it only moves (and O, l are rescaled) when a chunk's maximum
            // exceeds it by more than 2^8, so probabilities stay below 256.
            float m = -INFINITY, l = 0.f;
            int ci[3] = {0, 0, 0};
            uint32_t colbits = 0u;               // separable geometry: valid columns of one inner row
            int cached_c2 = -1;

            for (int c = 0; c < T.nch; ++c, ++gc) {
                // ---- validity words of this thread's two 32-column pieces ----
                uint32_t words[2];
                if (c >= T.nnb) {                // additional tokens: every live row sees the first n_extra columns
#pragma unroll
                    for (int pc = 0; pc < 2; ++pc)
                        words[pc] = valid_q ? low_bits(P.n_extra - ((c - T.nnb) * kChunk + 64 * team + 32 * pc)) : 0u;
                } else if constexpr (kInner > 0) {
                    if (ci[2] != cached_c2) {
                        cached_c2 = ci[2];
                        int lo2 = f[2] - ci[2] * kInner, hi2 = e[2] - ci[2] * kInner;
                        lo2 = lo2 > 0 ? lo2 : 0;
                        hi2 = hi2 < kInner ? hi2 : kInner;
                        colbits = hi2 > lo2 ? (low_bits(hi2 - lo2) << lo2) : 0u;
                    }
#pragma unroll
                    for (int pc = 0; pc < 2; ++pc) {
                        uint32_t w = 0u;
#pragma unroll
                        for (int t = 0; t < 32 / kInner; ++t) {
                            const int jj = 64 * team + 32 * pc + t * kInner;
                            const int j1 = (jj >> P.cb2_log) & (P.cb[1] - 1);
                            const int j0 = jj >> (P.cb2_log + P.cb1_log);
                            const int i0 = ci[0] * P.cb[0] + j0, i1 = ci[1] * P.cb[1] + j1;
                            if (i0 >= f[0] && i0 < e[0] && i1 >= f[1] && i1 < e[1]) w |= colbits << (t * kInner);
                        }
                        words[pc] = w;
                    }
                } else {
#pragma unroll
                    for (int pc = 0; pc < 2; ++pc) words[pc] = piece_word(P, ci, 2 * team + pc, f, e);
                }

                // ---- scores of this half into registers; S is free for the next chunk after that ----
                ok = ok && mbar_wait(bar_s, gc & 1, abort_flag);
                tc_fence_after();
                uint32_t s0[32], s1[32];
                const bool any0 = __any_sync(0xffffffffu, words[0] != 0u);
                const bool any1 = __any_sync(0xffffffffu, words[1] != 0u);
                if (any0) tmem_ld32(trow + kColS + 64 * team, s0);
                if (any1) tmem_ld32(trow + kColS + 64 * team + 32, s1);
                tmem_ld_wait();

                // ---- maximum over the valid columns of this half, then agree with the other half ----
                // columns outside the row's neighbourhood become -inf once, here
                float mc = -INFINITY;
                auto masked_max = [&](uint32_t (&s)[32], uint32_t w) {
                    float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
                    for (int i = 0; i < 32; i += 4) {
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            if (!((w >> (i + j)) & 1u)) s[i + j] = 0xff800000u;
                        m0 = fmaxf(m0, __uint_as_float(s[i]));
                        m1 = fmaxf(m1, __uint_as_float(s[i + 1]));
                        m2 = fmaxf(m2, __uint_as_float(s[i + 2]));
                        m3 = fmaxf(m3, __uint_as_float(s[i + 3]));
                    }
                    mc = fmaxf(mc, fmaxf(fmaxf(m0, m1), fmaxf(m2, m3)));
                };
                if (any0) masked_max(s0, words[0]);
                if (any1) masked_max(s1, words[1]);
                if (!ok) mc = -INFINITY;
                {
                    // Both halves must use one maximum.  Each publishes its own rounded up to bf16
                    // (any value >= the true maximum works as the stabiliser) and takes the larger.
                    uint32_t bits = __float_as_uint(mc);
                    bits = (mc >= 0.f) ? ((bits + 0xFFFFu) & 0xFFFF0000u) : (bits & 0xFFFF0000u);
                    xmax[team * 128 + row] = static_cast<uint16_t>(bits >> 16);
                    asm volatile("bar.sync %0, 64;" ::"r"(1 + quad) : "memory");
                    const uint32_t other = static_cast<uint32_t>(xmax[(1 - team) * 128 + row]) << 16;
                    mc = fmaxf(__uint_as_float(bits), __uint_as_float(other));
                }
                // S(c) is in registers and the partner's maximum has been read: the next scores may
                // land (they are what lets this thread overwrite its exchange slot again).
                tc_fence_before();
                mbar_arrive(bar_sr);

                // ---- P(c-1) V has finished: P may be rewritten, O may be rescaled ----
                if (c > 0) {
                    ok = ok && mbar_wait(bar_o, (gc - 1) & 1, abort_flag);
                    tc_fence_after();
                }
                bool grow = false;
                if (mc > -INFINITY) {
                    if (m == -INFINITY) m = mc;
                    else grow = (mc - m) * P.scale_log2 > 8.f;
                }
                if (__any_sync(0xffffffffu, grow)) {          // rare: both halves of a row decide alike
                    const float fac = grow ? fast_exp2((m - mc) * P.scale_log2) : 1.f;
#pragma unroll 1
                    for (int part = 0; part < CH / 16; ++part) {
                        uint32_t o[16];
                        tmem_ld16(trow + kColO + CH * team + 16 * part, o);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * fac);
                        tmem_st16(trow + kColO + CH * team + 16 * part, o);
                    }
                    l *= fac;
                    if (grow) m = mc;
                }
                const float mb = (m == -INFINITY) ? 0.f : m * P.scale_log2;

                // ---- probabilities -> TMEM (16-bit pairs), row sum of this half ----
                float r0 = 0.f, r1 = 0.f;
                auto probabilities = [&](const uint32_t (&s)[32], bool any, int pc) {
                    uint32_t packed[16];
                    if (any) {
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const float p0 = fast_exp2(fmaf(__uint_as_float(s[2 * i]), P.scale_log2, -mb));
                            const float p1 = fast_exp2(fmaf(__uint_as_float(s[2 * i + 1]), P.scale_log2, -mb));
                            r0 += p0;
                            r1 += p1;
                            packed[i] = cvt_pack<BF16>(p0, p1);
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 16; ++i) packed[i] = 0u;
                    }
                    tmem_st16(trow + kColP + 32 * team + 16 * pc, packed);
                };
                probabilities(s0, any0, 0);
                probabilities(s1, any1, 1);
                l += ok ? r0 + r1 : 0.f;
                tmem_st_wait();
                tc_fence_before();
                mbar_arrive(bar_sp);
                if (++ci[2] == T.nc[2]) { ci[2] = 0; if (++ci[1] == T.nc[1]) { ci[1] = 0; ++ci[0]; } }
            }

            // ---- all of P V is in O: combine the two halves' sums, normalise, write out ----
            ok = ok && mbar_wait(bar_o, (gc - 1) & 1, abort_flag);
            tc_fence_after();
            // The halves swap their row sums through two TMEM columns of the (now idle) P area; the
            // next tile's first chunk passes the pair's bar.sync again before it stores probabilities.
            tmem_st1(trow + kColP + team, __float_as_uint(l));
            tmem_st_wait();
            asm volatile("bar.sync %0, 64;" ::"r"(1 + quad) : "memory");
            {
                const bool live = valid_q && ok;
#pragma unroll
                for (int part = 0; part < CH / 32; ++part) {
                    uint32_t o[32], l_other = 0u;
                    if (part == 0) l_other = tmem_ld1(trow + kColP + (1 - team));
                    tmem_ld32(trow + kColO + CH * team + 32 * part, o);
                    tmem_ld_wait();
                    if (part == 0) l += __uint_as_float(l_other);
                    const float inv = (live && l > 0.f) ? 1.f / l : 0.f;
                    if (in_tensor) {
                        uint4* o4 = reinterpret_cast<uint4*>(out + out_row * DH + team * CH + 32 * part);
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            uint32_t w[4];
#pragma unroll
                            for (int j = 0; j < 4; ++j)
                                w[j] = cvt_pack<BF16>(__uint_as_float(o[8 * i + 2 * j]) * inv, __uint_as_float(o[8 * i + 2 * j + 1]) * inv);
                            o4[i] = make_uint4(w[0], w[1], w[2], w[3]);
                        }
                    }
                }
                // natural-log lse of scale * logits
                if (in_tensor && team == 0)
                    lse[out_row] = (live && l > 0.f) ? (m * P.scale_log2 + log2f(l)) * 0.6931471805599453f : 0.f;
            }
            if (tr && tid == 0) { tr[120] = t_begin; tr[121] = clock64(); tr = nullptr; }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 8) {
        tc_fence_after();
        tmem_dealloc(tmem, kTmemCols);
        if (lane == 0 && *abort_flag) atomicExch(P.status, 1);
    }
}

} // namespace

int tc_fused_fwd(int dtype, const Geo& g, const void* q, const void* k, const void* v, const void* ek,
                 const void* ev, void* out, void* lse, cudaStream_t s)
{
    if (!tc_eligible(dtype, g, q, k, v)) return -2;
    if (g.n_extra > 0 && ((reinterpret_cast<uintptr_t>(ek) | reinterpret_cast<uintptr_t>(ev)) & 15u)) return -2;
    Plan plan;
    if (!make_plan(g, plan)) return -2;
    const bool bf16 = dtype == 2;
    CUtensorMap mq, mk, mv, mek, mev;
    if (!encode_map(&mq, q, bf16, plan.p, g.Hq, g.D, g.qs, plan.box_q) ||
        !encode_map(&mk, k, bf16, plan.p, g.Hkv, g.D, g.ks, plan.box_kv) ||
        !encode_map(&mv, v, bf16, plan.p, g.Hkv, g.Dv, g.vs, plan.box_kv))
        return -2;
    mek = mk; mev = mv;                      // placeholders when there are no additional tokens
    if (g.n_extra > 0 && (!encode_extra_map(&mek, ek, bf16, g.B, g.n_extra, g.Hkv, g.D, kChunk) ||
                          !encode_extra_map(&mev, ev, bf16, g.B, g.n_extra, g.Hkv, g.Dv, kChunk)))
        return -2;
    plan.p.status = status_ptr();
    plan.p.trace = trace_ptr();
    if (!plan.p.status) return -2;
    int ngroups = 1;
    for (int a = 0; a < 3; ++a) ngroups *= plan.p.dil[a];
    if (plan.p.work_q == 0) return 0;
    const dim3 grid(persistent_grid(plan.p.work_q, g.D == 64 ? 2 : 1));
    cudaError_t err;
    auto launch = [&](auto dh, auto bf, auto inner) {
        constexpr int kDh = decltype(dh)::value;
        constexpr bool kBf = decltype(bf)::value;
        constexpr int kInner = decltype(inner)::value;
        using SM = SmemMap<kDh>;
        static bool once = false;
        if (!once) {
            cudaFuncSetAttribute(tc_fwd_kernel<kDh, kBf, kInner>, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::kTotal);
            once = true;
        }
        tc_fwd_kernel<kDh, kBf, kInner><<<grid, kThreads, SM::kTotal, s>>>(mq, mk, mv, mek, mev, plan.p, (uint16_t*)out, (float*)lse);
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
    if (g.D == 64) by_type(std::integral_constant<int, 64>{});
    else by_type(std::integral_constant<int, 128>{});
    err = cudaGetLastError();
    tc_count_launch();
    return err == cudaSuccess ? 0 : (int)err;
}

static unsigned long long g_tc_launches = 0;
void tc_count_launch() { ++g_tc_launches; }
unsigned long long tc_launch_count() { return g_tc_launches; }

int tc_device_status()
{
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(int)) != cudaSuccess) return -1;
    return v;
}

} // namespace natten
