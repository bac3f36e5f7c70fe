// Split neighbourhood products on tcgen05 tensor cores (sm_100a).
//
// scores kernel:  out[row, slot] = scale * <x[row], y[key of slot]>      (QK forward: x = q, y = k;
//                                                                          AV backward w.r.t. attn: x = dout, y = v)
// One CTA handles a box of 128 rows of one (batch, head); the union of their neighbourhoods is a box
// of keys walked in chunks of 128 (the same geometry as the fused forward).  Per chunk S = X Y^T on
// the tensor cores (operands staged by TMA, accumulator in TMEM); the threads read S and scatter the
// entries that belong to each row's window into a [128 x slots] tile in shared memory, which is
// written out with coalesced stores when the tile is complete.  Slots whose key is masked (causal
// start of an axis) keep the fill value (-inf for logits, 0 for a gradient).
#include "tc_kernels.cuh"

#include "tc_plan.cuh"

#include <type_traits>

namespace natten {

using namespace tc;
using namespace tcplan;

namespace {

constexpr int kThreads = 288;            // 8 scatter warps + TMA/MMA warp
constexpr int kStages = 3;

template <int DH>
struct SmemS {
    static constexpr int kHalves = DH / 64;
    static constexpr int kHalf = kTileRows * 128;
    static constexpr int kTile = kHalf * kHalves;
    static constexpr int kX = 0;
    static constexpr int kY = kX + kTile;                 // [kStages]
    static constexpr int kBar = kY + kStages * kTile;     // barriers, flags: 128 bytes
    static constexpr int kColSlot = kBar + 128;           // [128] int: slot offset of a chunk column
    static constexpr int kRowOut = kColSlot + 512;        // [128] long long: output row or -1
    static constexpr int kOut = kRowOut + 1024;           // [128][slots] 16-bit
};

__device__ __forceinline__ int tc_window_start(int p, int L, int K) { return window_start(p, L, K, 1); }

// Geometry of one CTA: a box of 128 rows of one dilation group, and the key box their windows cover.
struct SplitGeo {
    int rg[3], origin[3], Lp[3], lo[3], nc[3], x0[3], sx[3], nq[3];
    int nch;
};

__device__ __forceinline__ bool split_cta_geometry(const TcParams& P, unsigned bx, int b, SplitGeo& G)
{
    bool active = cta_geometry(P, bx, b, G.rg, G.origin, G.Lp);
#pragma unroll
    for (int a = 0; a < 3; ++a) {
        G.sx[a] = P.qstep[a];
        G.x0[a] = P.qx0[a][G.rg[a]];
        if (G.x0[a] < 0) { G.nq[a] = 0; G.x0[a] = 0; }
        else if (G.sx[a] == 1) G.nq[a] = G.Lp[a];
        else G.nq[a] = G.x0[a] < G.Lp[a] ? (G.Lp[a] - G.x0[a] + G.sx[a] - 1) / G.sx[a] : 0;
        if (G.origin[a] >= G.nq[a]) active = false;
    }
    if (!active) return false;               // without per-sample extents every output row belongs to an active tile
    G.nch = 1;
#pragma unroll
    for (int a = 0; a < 3; ++a) {
        const int lastq = G.origin[a] + P.tile[a] - 1 < G.nq[a] - 1 ? G.origin[a] + P.tile[a] - 1 : G.nq[a] - 1;
        const int xf = G.x0[a] + G.sx[a] * G.origin[a], xl = G.x0[a] + G.sx[a] * lastq;
        G.lo[a] = P.causal[a] ? xf - (P.K[a] - 1) : tc_window_start(xf, G.Lp[a], P.K[a]);
        const int hi = P.causal[a] ? xl : tc_window_start(xl, G.Lp[a], P.K[a]) + P.K[a] - 1;
        G.nc[a] = chunks_along(P, a, hi - G.lo[a] + 1);
        G.nch *= G.nc[a];
    }
    return true;
}

// One row of the tile: valid column box [f, e), first slot fs (box coordinates), flat output position.
__device__ __forceinline__ bool split_row(const TcParams& P, const SplitGeo& G, int row, int (&f)[3], int (&e)[3],
                                          int (&fs)[3], long long& oflat, long long& pflat)
{
    int qi[3];
    row_offsets(P, row, qi);
    bool valid = true;
    oflat = 0;
    pflat = 0;
#pragma unroll
    for (int a = 0; a < 3; ++a) {
        const int qa = G.origin[a] + qi[a];
        const int xq = G.x0[a] + G.sx[a] * qa;
        const int pa = G.rg[a] + P.dil[a] * xq;
        if (qa >= G.nq[a]) valid = false;
        oflat = oflat * P.O[a] + (P.st[a] == 1 ? pa : pa / P.st[a]);
        pflat = pflat * P.L[a] + pa;
        const int first = P.causal[a] ? xq - (P.K[a] - 1) : tc_window_start(xq, G.Lp[a], P.K[a]);
        fs[a] = first - G.lo[a];
        f[a] = (first > 0 ? first : 0) - G.lo[a];
        e[a] = (first + P.K[a] < G.Lp[a] ? first + P.K[a] : G.Lp[a]) - G.lo[a];
    }
    if (!valid) { e[0] = f[0]; e[1] = f[1]; e[2] = f[2]; }
    return valid;
}

// kInner = 16: the chunk's innermost extent is 16 columns (every 16 columns of a chunk are one inner row whose
// slots are consecutive: static offsets from one pointer per row); 0: any geometry (slot table per column).
template <int DH, bool BF16, int kInner>
__global__ void __launch_bounds__(kThreads, (DH == 64 ? 2 : 1))
tc_scores_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmY,
                 const __grid_constant__ TcParams P, uint16_t* __restrict__ out, float scale, uint32_t fill16,
                 int ktot, const uint16_t* __restrict__ rpb, int rpb_table)
{
    using SM = SmemS<DH>;
    extern __shared__ __align__(1024) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = blockIdx.y, b = blockIdx.z, hk = h / P.group;
    const int quad = warp & 3, team = (warp >> 2) & 1;        // scatter warps: TMEM lane quadrant, column half
    const int prior_abort = *reinterpret_cast<volatile int*>(P.status);

    // ---- CTA geometry (same as the fused forward; queries may sit on a strided lattice) ----
    int rg[3], origin[3], Lp[3], lo[3], nc[3], x0[3], sx[3], nq[3], nqf[3];
    bool cta_active = cta_geometry(P, blockIdx.x, b, rg, origin, Lp);
#pragma unroll
    for (int a = 0; a < 3; ++a) {
        sx[a] = P.qstep[a];
        x0[a] = P.qx0[a][rg[a]];
        const int lpf = (P.L[a] - rg[a] + P.dil[a] - 1) / P.dil[a];
        if (x0[a] < 0) {
            nq[a] = 0; nqf[a] = 0; x0[a] = 0;
        } else if (sx[a] == 1) {
            nq[a] = Lp[a];
            nqf[a] = rg[a] < P.L[a] ? lpf : 0;
        } else {
            nq[a] = x0[a] < Lp[a] ? (Lp[a] - x0[a] + sx[a] - 1) / sx[a] : 0;
            nqf[a] = x0[a] < lpf ? (lpf - x0[a] + sx[a] - 1) / sx[a] : 0;
        }
        if (origin[a] >= nq[a]) cta_active = false;
    }
    if (!cta_active) return;                 // without per-sample extents every output row belongs to an active tile
    int nch = 1;
#pragma unroll
    for (int a = 0; a < 3; ++a) {
        const int lastq = origin[a] + P.tile[a] - 1 < nq[a] - 1 ? origin[a] + P.tile[a] - 1 : nq[a] - 1;
        const int xf = x0[a] + sx[a] * origin[a], xl = x0[a] + sx[a] * lastq;
        lo[a] = P.causal[a] ? xf - (P.K[a] - 1) : tc_window_start(xf, Lp[a], P.K[a]);
        const int hi = P.causal[a] ? xl : tc_window_start(xl, Lp[a], P.K[a]) + P.K[a] - 1;
        nc[a] = chunks_along(P, a, hi - lo[a] + 1);
        nch *= nc[a];
    }

    const uint32_t sbase = smem_u32(smem);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + SM::kBar + 64);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + SM::kBar + 72);
    int* colslot = reinterpret_cast<int*>(smem + SM::kColSlot);
    long long* rowout = reinterpret_cast<long long*>(smem + SM::kRowOut);
    uint16_t* tile = reinterpret_cast<uint16_t*>(smem + SM::kOut);
    // relative position bias (optional): per row the first bias entry of its window, per slot its offset from there
    int* rowpb = reinterpret_cast<int*>(smem + SM::kOut + ((kTileRows * ktot * 2 + 15) & ~15));
    int* slotpb = rowpb + kTileRows;
    const uint32_t bar_x = sbase + SM::kBar + 0;
    const uint32_t bar_y = sbase + SM::kBar + 8;        // [3]
    const uint32_t bar_s = sbase + SM::kBar + 32;
    const uint32_t bar_sp = sbase + SM::kBar + 40;

    int ld[3] = {0, 0, 0}, loaded = 0;
    auto issue_y = [&]() {
        const int s = loaded % kStages;
        const uint32_t bar = bar_y + 8 * s;
        mbar_expect_tx(bar, SM::kTile);
        int X[3];
#pragma unroll
        for (int a = 0; a < 3; ++a) X[a] = rg[a] + P.dil[a] * (lo[a] + ld[a] * P.cb[a]);
#pragma unroll
        for (int hf = 0; hf < SM::kHalves; ++hf)
            tma_load_5d(sbase + SM::kY + s * SM::kTile + hf * SM::kHalf, &tmY, bar, hk * DH + 64 * hf, X[2], X[1], X[0], b);
        if (++ld[2] == nc[2]) { ld[2] = 0; if (++ld[1] == nc[1]) { ld[1] = 0; ++ld[0]; } }
        ++loaded;
    };
    if (warp == 8) {
        if (lane == 0) {
            *abort_flag = ((sbase & 1023u) || prior_abort) ? 1 : 0;
            mbar_init(bar_x, 1);
            for (int s = 0; s < kStages; ++s) mbar_init(bar_y + 8 * s, 1);
            mbar_init(bar_s, 1);
            mbar_init(bar_sp, 256);
            mbar_init_fence();
            fence_async_smem();
            if (!*abort_flag) {
                mbar_expect_tx(bar_x, SM::kTile);
#pragma unroll
                for (int hf = 0; hf < SM::kHalves; ++hf)
                    tma_load_5d(sbase + SM::kX + hf * SM::kHalf, &tmX, bar_x, h * DH + 64 * hf,
                                rg[2] + P.dil[2] * (x0[2] + sx[2] * origin[2]), rg[1] + P.dil[1] * (x0[1] + sx[1] * origin[1]),
                                rg[0] + P.dil[0] * (x0[0] + sx[0] * origin[0]), b);
                for (int c = 0; c < nch && c < kStages; ++c) issue_y();
            }
        }
        __syncwarp();
        tmem_alloc(smem_u32(tmem_slot), 128);
    }
    // ---- per-thread row; shared tables; the output tile starts filled with the mask value ----
    int f[3] = {0, 0, 0}, e[3] = {0, 0, 0}, fs[3] = {0, 0, 0};
    const int row = quad * 32 + lane;
    if (warp < 8) {
        int qi[3];
        row_offsets(P, row, qi);
        bool valid_q = true;
        long long oflat = 0;
#pragma unroll
        for (int a = 0; a < 3; ++a) {
            const int qa = origin[a] + qi[a];
            const int xq = x0[a] + sx[a] * qa;
            const int pa = rg[a] + P.dil[a] * xq;
            if (qa >= nq[a]) valid_q = false;
            oflat = oflat * P.O[a] + (P.st[a] == 1 ? pa : pa / P.st[a]);
            const int first = P.causal[a] ? xq - (P.K[a] - 1) : tc_window_start(xq, Lp[a], P.K[a]);
            fs[a] = first - lo[a];                                        // slot 0 of the axis, in box coordinates
            f[a] = (first > 0 ? first : 0) - lo[a];
            e[a] = (first + P.K[a] < Lp[a] ? first + P.K[a] : Lp[a]) - lo[a];
        }
        if (!valid_q) { e[0] = f[0]; e[1] = f[1]; e[2] = f[2]; }
        if (team == 0) rowout[row] = valid_q ? (((long long)b * P.otot + oflat) * P.Hq + h) * ktot : -1;   // element offset
        if (rpb) {                               // unit stride, no causal axis: the bias window start of the reference
            if (team == 0) {
                int pbi = 0;
#pragma unroll
                for (int a = 0; a < 3; ++a) {
                    const int pa = rg[a] + P.dil[a] * (x0[a] + sx[a] * (origin[a] + qi[a]));
                    const int K = P.K[a], nh = K / 2, L = P.L[a], d = P.dil[a];
                    int pb;
                    if (d <= 1) pb = nh + (pa < nh ? nh - pa : (pa + nh >= L ? L - pa - 1 - nh : 0));
                    else pb = pa - nh * d < 0 ? K - 1 - pa / d : (pa + nh * d >= L ? (L - pa - 1) / d : nh);
                    pbi = pbi * (2 * K - 1) + pb;
                }
                rowpb[row] = pbi;
            }
            for (int j = tid; j < ktot; j += 256) {
                int rem = j, off = 0, mul = 1;
#pragma unroll
                for (int a = 2; a >= 0; --a) {
                    off += (rem % P.K[a]) * mul;
                    rem /= P.K[a];
                    mul *= 2 * P.K[a] - 1;
                }
                slotpb[j] = off;
            }
        }
        // column jj of a chunk sits at box offset (j0, j1, j2): its slot relative to the chunk's first column
        if (tid < 128) {
            const int j2 = tid & (P.cb[2] - 1);
            const int j1 = (tid >> P.cb2_log) & (P.cb[1] - 1);
            const int j0 = tid >> (P.cb2_log + P.cb1_log);
            colslot[tid] = (j0 * P.K[1] + j1) * P.K[2] + j2;
        }
        for (int j = team; j < ktot; j += 2) tile[row * ktot + j] = static_cast<uint16_t>(fill16);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 8) {
        // the warp runs the loop converged; the tensor-core instructions execute on an elected lane
        const uint32_t leader = elect_one();
        if (!*abort_flag) {
            constexpr uint32_t idesc = instr_desc(BF16 ? 1 : 0, kChunk, 0, 0);
            const uint64_t dx0 = smem_desc(sbase + SM::kX, 16, 1024);
            auto issue_s = [&](int c) {
                const uint64_t dy0 = smem_desc(sbase + SM::kY + (c % kStages) * SM::kTile, 16, 1024);
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < DH / 16; ++ks) {
                    const uint32_t off = ((ks / 4) * SM::kHalf + (ks % 4) * 32) >> 4;
                    mma_ss_e(tmem, dx0 + off, dy0 + off, idesc, ks > 0, leader);
                }
                mma_commit_e(bar_s, leader);
            };
            bool ok = mbar_wait(bar_x, 0, abort_flag, P.wait_budget) && mbar_wait(bar_y, 0, abort_flag, P.wait_budget);
            if (ok) issue_s(0);
            for (int c = 0; c < nch && ok; ++c) {
                ok = mbar_wait(bar_s, c & 1, abort_flag, P.wait_budget);            // the product is done: its Y stage is free
                if (!ok) break;
                if (c + kStages < nch && leader) issue_y();
                __syncwarp();
                ok = mbar_wait(bar_sp, c & 1, abort_flag, P.wait_budget);           // S(c) read by every thread
                if (!ok) break;
                if (c + 1 < nch) {
                    ok = mbar_wait(bar_y + 8 * ((c + 1) % kStages), ((c + 1) / kStages) & 1, abort_flag, P.wait_budget);
                    if (!ok) break;
                    issue_s(c + 1);
                }
            }
        }
    } else {
        const uint32_t trow = tmem + (static_cast<uint32_t>(quad * 32) << 16);
        uint16_t* myrow = tile + row * ktot;
        bool ok = true;
        int ci[3] = {0, 0, 0};
        for (int c = 0; c < nch; ++c) {
            uint32_t words[2];
#pragma unroll
            for (int pc = 0; pc < 2; ++pc) words[pc] = piece_word(P, ci, 2 * team + pc, f, e);
            // slot of the chunk's first column for this row
            const int base = ((ci[0] * P.cb[0] - fs[0]) * P.K[1] + (ci[1] * P.cb[1] - fs[1])) * P.K[2] + (ci[2] * P.cb[2] - fs[2]);
            ok = ok && mbar_wait(bar_s, c & 1, abort_flag, P.wait_budget);
            tc_fence_after();
            uint16_t* dstp = myrow + base;        // slot 0 of this chunk's first column, for this row
#pragma unroll
            for (int pc = 0; pc < 2; ++pc) {
                if (!__any_sync(0xffffffffu, words[pc] != 0u)) continue;
                uint32_t s[32];
                tmem_ld32(trow + 64 * team + 32 * pc, s);
                tmem_ld_wait();
                if (ok && kInner == 16) {
                    // two inner rows of 16 columns: column j2 of a row goes to slot (row's first slot) + j2
#pragma unroll
                    for (int rr = 0; rr < 2; ++rr) {
                        const uint32_t bits = (words[pc] >> (16 * rr)) & 0xFFFFu;
                        if (bits == 0u) continue;
                        const int r = 4 * team + 2 * pc + rr;                    // inner row of the chunk
                        const int i0 = ci[0] * P.cb[0] + (r >> P.cb1_log), i1 = ci[1] * P.cb[1] + (r & (P.cb[1] - 1));
                        uint16_t* rowp = myrow + ((i0 - fs[0]) * P.K[1] + (i1 - fs[1])) * P.K[2] + (ci[2] * 16 - fs[2]);
#pragma unroll
                        for (int i = 0; i < 16; i += 2) {
                            const uint32_t both = cvt_pack<BF16>(__uint_as_float(s[16 * rr + i]) * scale, __uint_as_float(s[16 * rr + i + 1]) * scale);
                            if ((bits >> i) & 1u) rowp[i] = static_cast<uint16_t>(both & 0xFFFFu);
                            if ((bits >> (i + 1)) & 1u) rowp[i + 1] = static_cast<uint16_t>(both >> 16);
                        }
                    }
                } else if (ok) {
                    const int* cs = colslot + 64 * team + 32 * pc;
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {     // pairs: one conversion for two columns
                        const uint32_t both = cvt_pack<BF16>(__uint_as_float(s[i]) * scale, __uint_as_float(s[i + 1]) * scale);
                        if ((words[pc] >> i) & 1u) dstp[cs[i]] = static_cast<uint16_t>(both & 0xFFFFu);
                        if ((words[pc] >> (i + 1)) & 1u) dstp[cs[i + 1]] = static_cast<uint16_t>(both >> 16);
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(bar_sp);
            if (++ci[2] == nc[2]) { ci[2] = 0; if (++ci[1] == nc[1]) { ci[1] = 0; ++ci[0]; } }
        }
        // ---- the tile is complete: coalesced copy to the output ----
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (ok) {
            // consecutive threads copy consecutive elements of a row: 256 elements ahead = dr rows and dj slots
            int r = tid / ktot, j = tid - r * ktot;
            const int dr = 256 / ktot, dj = 256 - dr * ktot;
            const int total = kTileRows * ktot;
            for (int idx = tid; idx < total; idx += 256) {
                const long long off = rowout[r];
                if (off >= 0) {
                    uint16_t v = tile[idx];
                    if (rpb) {                   // masked slots hold -inf and stay -inf
                        const uint32_t bv = rpb[(long long)h * rpb_table + rowpb[r] + slotpb[j]];
                        const float x = BF16 ? __uint_as_float(static_cast<uint32_t>(v) << 16) : __half2float(__ushort_as_half(v));
                        const float y = BF16 ? __uint_as_float(bv << 16) : __half2float(__ushort_as_half(static_cast<unsigned short>(bv)));
                        v = static_cast<uint16_t>(cvt_pack<BF16>(x + y, 0.f) & 0xFFFFu);
                    }
                    out[off + j] = v;
                }
                r += dr;
                j += dj;
                if (j >= ktot) { j -= ktot; ++r; }
            }
        }
    }

    if (*abort_flag) abort_grace_sleep();       // loads of a wait that gave up may still be landing
    tc_fence_before();
    __syncthreads();
    if (warp == 8) {
        tc_fence_after();
        tmem_dealloc(tmem, 128);
        if (lane == 0 && *abort_flag) atomicExch(P.status, 1);
    }
}

template <int DH, bool BF16, int kInner>
int launch_scores_inner(const Plan& plan, const CUtensorMap& mx, const CUtensorMap& my, const Geo& g, void* out,
                        float scale, bool neg_inf, cudaStream_t s, const void* rpb, int rpb_table);

template <int DH, bool BF16>
int launch_scores(const Plan& plan, const CUtensorMap& mx, const CUtensorMap& my, const Geo& g, void* out,
                  float scale, bool neg_inf, cudaStream_t s, const void* rpb, int rpb_table)
{
    return plan.p.cb[2] == 16 ? launch_scores_inner<DH, BF16, 16>(plan, mx, my, g, out, scale, neg_inf, s, rpb, rpb_table)
                              : launch_scores_inner<DH, BF16, 0>(plan, mx, my, g, out, scale, neg_inf, s, rpb, rpb_table);
}

template <int DH, bool BF16, int kInner>
int launch_scores_inner(const Plan& plan, const CUtensorMap& mx, const CUtensorMap& my, const Geo& g, void* out,
                        float scale, bool neg_inf, cudaStream_t s, const void* rpb, int rpb_table)
{
    using SM = SmemS<DH>;
    const size_t smem = (size_t)SM::kOut + (((size_t)kTileRows * g.ktot * 2 + 15) & ~(size_t)15) + (rpb ? 4 * (kTileRows + (size_t)g.ktot) : 0);
    if (smem > kMaxDynamicSmem) return -2;
    if (ensure_dynamic_smem((const void*)tc_scores_kernel<DH, BF16, kInner>, kMaxDynamicSmem) != cudaSuccess) {
        cudaGetLastError();
        return -2;
    }
    int ngroups = 1;
    for (int a = 0; a < 3; ++a) ngroups *= plan.p.grp_n[a];
    const dim3 grid((unsigned)(plan.p.ntiles * ngroups), (unsigned)g.Hq, (unsigned)g.B);
    const uint32_t fill = neg_inf ? (BF16 ? 0xFF80u : 0xFC00u) : 0u;
    tc_scores_kernel<DH, BF16, kInner><<<grid, kThreads, smem, s>>>(mx, my, plan.p, (uint16_t*)out, scale, fill, g.ktot,
                                                                   (const uint16_t*)rpb, rpb_table);
    tc_count_launch();
    const cudaError_t err = cudaGetLastError();
    return err == cudaSuccess ? 0 : (int)err;
}

// ---------------------------------------------------------------------------
// apply kernel:  out[row] = scale * sum_slot w[row, slot] * y[key of slot]     (AV forward: w = attn, y = v;
//                                                                                QK backward w.r.t. q: w = dlogits, y = k)
// The CTA's [128 x slots] block of w is staged in shared memory; per chunk of 128 keys the threads
// gather the weights of the columns inside each row's window into a dense 16-bit P tile in TMEM
// (two buffers), and O += P Y runs on the tensor cores with Y read MN-major, as in the fused forward.
// ---------------------------------------------------------------------------
template <int DH>
struct SmemA {
    static constexpr int kHalves = DH / 64;
    static constexpr int kHalf = kTileRows * 128;
    static constexpr int kTile = kHalf * kHalves;
    static constexpr int kY = 0;                          // [kStages]
    static constexpr int kBar = kY + kStages * kTile;     // barriers, flags: 128 bytes
    static constexpr int kColSlot = kBar + 128;
    static constexpr int kRowOut = kColSlot + 512;        // [128] long long: row of w / out, or -1
    static constexpr int kW = kRowOut + 1024;             // [128][slots] 16-bit
    static constexpr uint32_t kColP = 0;                  // two buffers of 64 columns
    static constexpr uint32_t kColO = 128;
    static constexpr uint32_t kTmemCols = 256;
};

template <int DH, bool BF16, int kInner>
__global__ void __launch_bounds__(kThreads, (DH == 64 ? 2 : 1))
tc_apply_kernel(const __grid_constant__ CUtensorMap tmY, const __grid_constant__ TcParams P,
                const uint16_t* __restrict__ w, uint16_t* __restrict__ out, float scale, int ktot,
                int out_by_position)
{
    using SM = SmemA<DH>;
    constexpr int CH = DH / 2;
    extern __shared__ __align__(1024) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = blockIdx.y, b = blockIdx.z, hk = h / P.group;
    const int quad = warp & 3, team = (warp >> 2) & 1;
    const int prior_abort = *reinterpret_cast<volatile int*>(P.status);
    SplitGeo G;
    if (!split_cta_geometry(P, blockIdx.x, b, G)) return;
    const int nch = G.nch;

    const uint32_t sbase = smem_u32(smem);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + SM::kBar + 64);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + SM::kBar + 72);
    int* colslot = reinterpret_cast<int*>(smem + SM::kColSlot);
    long long* rowout = reinterpret_cast<long long*>(smem + SM::kRowOut);
    uint16_t* wt = reinterpret_cast<uint16_t*>(smem + SM::kW);
    const uint32_t bar_y = sbase + SM::kBar + 0;         // [3] Y chunk landed
    const uint32_t bar_p = sbase + SM::kBar + 48;        // [2] P buffer b stored by every thread
    const uint32_t bar_o = sbase + SM::kBar + 32;        // [2] the MMAs that read P buffer b have finished

    int ld[3] = {0, 0, 0}, loaded = 0;
    auto issue_y = [&]() {
        const int s = loaded % kStages;
        const uint32_t bar = bar_y + 8 * s;
        mbar_expect_tx(bar, SM::kTile);
        int X[3];
#pragma unroll
        for (int a = 0; a < 3; ++a) X[a] = G.rg[a] + P.dil[a] * (G.lo[a] + ld[a] * P.cb[a]);
#pragma unroll
        for (int hf = 0; hf < SM::kHalves; ++hf)
            tma_load_5d(sbase + SM::kY + s * SM::kTile + hf * SM::kHalf, &tmY, bar, hk * DH + 64 * hf, X[2], X[1], X[0], b);
        if (++ld[2] == G.nc[2]) { ld[2] = 0; if (++ld[1] == G.nc[1]) { ld[1] = 0; ++ld[0]; } }
        ++loaded;
    };
    if (warp == 8) {
        if (lane == 0) {
            *abort_flag = ((sbase & 1023u) || prior_abort) ? 1 : 0;
            for (int s = 0; s < kStages; ++s) mbar_init(bar_y + 8 * s, 1);
            mbar_init(bar_p, 256);
            mbar_init(bar_p + 8, 256);
            mbar_init(bar_o, 1);
            mbar_init(bar_o + 8, 1);
            mbar_init_fence();
            fence_async_smem();
            if (!*abort_flag)
                for (int c = 0; c < nch && c < kStages; ++c) issue_y();
        }
        __syncwarp();
        tmem_alloc(smem_u32(tmem_slot), SM::kTmemCols);
    }
    int f[3], e[3], fs[3];
    const int row = quad * 32 + lane;
    long long orow = -1;
    if (warp < 8) {
        long long oflat, pflat;
        const bool valid = split_row(P, G, row, f, e, fs, oflat, pflat);
        const long long wrow = ((long long)b * P.otot + oflat) * P.Hq + h;          // row of w (by output position)
        orow = out_by_position ? ((long long)b * P.ltot + pflat) * P.Hq + h : wrow;
        if (!valid) orow = -1;
        if (team == 0) rowout[row] = valid ? wrow * ktot : -1;                      // element offset of the row of w
        if (tid < 128) {
            const int j2 = tid & (P.cb[2] - 1);
            const int j1 = (tid >> P.cb2_log) & (P.cb[1] - 1);
            const int j0 = tid >> (P.cb2_log + P.cb1_log);
            colslot[tid] = (j0 * P.K[1] + j1) * P.K[2] + j2;
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 8) {
        // the warp runs the loop converged; the tensor-core instructions execute on an elected lane
        const uint32_t leader = elect_one();
        if (!*abort_flag) {
            constexpr uint32_t idesc = instr_desc(BF16 ? 1 : 0, DH, 0, 1);      // A = P from TMEM, B = Y MN-major
            bool ok = true;
            for (int c = 0; c < nch && ok; ++c) {
                ok = mbar_wait(bar_y + 8 * (c % kStages), (c / kStages) & 1, abort_flag, P.wait_budget) &&
                     mbar_wait(bar_p + 8 * (c & 1), (c >> 1) & 1, abort_flag, P.wait_budget);
                if (!ok) break;
                const uint64_t dy0 = smem_desc(sbase + SM::kY + (c % kStages) * SM::kTile, SM::kHalf, 1024);
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < kChunk / 16; ++ks)
                    mma_ts_e(tmem + SM::kColO, tmem + SM::kColP + 64 * (c & 1) + 8 * ks, dy0 + 128 * ks, idesc, c > 0 || ks > 0, leader);
                mma_commit_e(bar_o + 8 * (c & 1), leader);
                if (c >= 1 && c + 2 < nch) {             // the product before this one is done: its Y stage is free
                    ok = mbar_wait(bar_o + 8 * ((c - 1) & 1), ((c - 1) >> 1) & 1, abort_flag, P.wait_budget);
                    if (!ok) break;
                    if (leader) issue_y();
                    __syncwarp();
                }
            }
        }
    } else {
        const uint32_t trow = tmem + (static_cast<uint32_t>(quad * 32) << 16);
        // ---- stage this tile's weights: rows are contiguous runs of `ktot` values ----
        {
            int r = tid / ktot, j = tid - r * ktot;
            const int dr = 256 / ktot, dj = 256 - dr * ktot;
            const int total = kTileRows * ktot;
            for (int idx = tid; idx < total; idx += 256) {
                const long long off = rowout[r];
                wt[idx] = off >= 0 ? w[off + j] : static_cast<uint16_t>(0);
                r += dr;
                j += dj;
                if (j >= ktot) { j -= ktot; ++r; }
            }
        }
        asm volatile("bar.sync 1, 256;" ::: "memory");
        const uint16_t* myrow = wt + row * ktot;
        bool ok = true;
        int ci[3] = {0, 0, 0};
        for (int c = 0; c < nch; ++c) {
            uint32_t words[2];
#pragma unroll
            for (int pc = 0; pc < 2; ++pc) words[pc] = piece_word(P, ci, 2 * team + pc, f, e);
            const int base = ((ci[0] * P.cb[0] - fs[0]) * P.K[1] + (ci[1] * P.cb[1] - fs[1])) * P.K[2] + (ci[2] * P.cb[2] - fs[2]);
            const uint16_t* srcp = myrow + base;  // slot 0 of this chunk's first column, for this row
            // P buffer c & 1 was last read by the product of chunk c - 2
            if (c >= 2) {
                ok = ok && mbar_wait(bar_o + 8 * (c & 1), ((c - 2) >> 1) & 1, abort_flag, P.wait_budget);
                tc_fence_after();
            }
#pragma unroll
            for (int pc = 0; pc < 2; ++pc) {
                uint32_t packed[16];
                if (kInner == 16 && __any_sync(0xffffffffu, words[pc] != 0u)) {
                    // two inner rows of 16 columns: column j2 of a row reads slot (row's first slot) + j2
#pragma unroll
                    for (int rr = 0; rr < 2; ++rr) {
                        const uint32_t bits = (words[pc] >> (16 * rr)) & 0xFFFFu;
                        const int r = 4 * team + 2 * pc + rr;                    // inner row of the chunk
                        const int i0 = ci[0] * P.cb[0] + (r >> P.cb1_log), i1 = ci[1] * P.cb[1] + (r & (P.cb[1] - 1));
                        const uint16_t* rowp = myrow + ((i0 - fs[0]) * P.K[1] + (i1 - fs[1])) * P.K[2] + (ci[2] * 16 - fs[2]);
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            uint32_t lo16 = 0u, hi16 = 0u;
                            if ((bits >> (2 * i)) & 1u) lo16 = rowp[2 * i];
                            if ((bits >> (2 * i + 1)) & 1u) hi16 = rowp[2 * i + 1];
                            packed[8 * rr + i] = lo16 | (hi16 << 16);
                        }
                    }
                } else if (__any_sync(0xffffffffu, words[pc] != 0u)) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const int c0 = 64 * team + 32 * pc + 2 * i;
                        uint32_t lo16 = 0u, hi16 = 0u;
                        if ((words[pc] >> (2 * i)) & 1u) lo16 = srcp[colslot[c0]];
                        if ((words[pc] >> (2 * i + 1)) & 1u) hi16 = srcp[colslot[c0 + 1]];
                        packed[i] = lo16 | (hi16 << 16);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 16; ++i) packed[i] = 0u;
                }
                tmem_st16(trow + SM::kColP + 64 * (c & 1) + 32 * team + 16 * pc, packed);
            }
            tmem_st_wait();
            tc_fence_before();
            mbar_arrive(bar_p + 8 * (c & 1));
            if (++ci[2] == G.nc[2]) { ci[2] = 0; if (++ci[1] == G.nc[1]) { ci[1] = 0; ++ci[0]; } }
        }
        // ---- every product is in O: scale, write out this thread's channels ----
        ok = ok && mbar_wait(bar_o + 8 * ((nch - 1) & 1), ((nch - 1) >> 1) & 1, abort_flag, P.wait_budget);
        tc_fence_after();
#pragma unroll
        for (int part = 0; part < CH / 32; ++part) {
            uint32_t o[32];
            tmem_ld32(trow + SM::kColO + CH * team + 32 * part, o);
            tmem_ld_wait();
            if (orow >= 0 && ok) {
                uint4* o4 = reinterpret_cast<uint4*>(out + orow * DH + team * CH + 32 * part);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    uint32_t x[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        x[j] = cvt_pack<BF16>(__uint_as_float(o[8 * i + 2 * j]) * scale, __uint_as_float(o[8 * i + 2 * j + 1]) * scale);
                    o4[i] = make_uint4(x[0], x[1], x[2], x[3]);
                }
            }
        }
    }

    if (*abort_flag) abort_grace_sleep();       // loads of a wait that gave up may still be landing
    tc_fence_before();
    __syncthreads();
    if (warp == 8) {
        tc_fence_after();
        tmem_dealloc(tmem, SM::kTmemCols);
        if (lane == 0 && *abort_flag) atomicExch(P.status, 1);
    }
}

template <int DH, bool BF16, int kInner>
int launch_apply_inner(const Plan& plan, const CUtensorMap& my, const Geo& g, const void* w, void* out, float scale,
                       bool out_by_position, cudaStream_t s);

template <int DH, bool BF16>
int launch_apply(const Plan& plan, const CUtensorMap& my, const Geo& g, const void* w, void* out, float scale,
                 bool out_by_position, cudaStream_t s)
{
    return plan.p.cb[2] == 16 ? launch_apply_inner<DH, BF16, 16>(plan, my, g, w, out, scale, out_by_position, s)
                              : launch_apply_inner<DH, BF16, 0>(plan, my, g, w, out, scale, out_by_position, s);
}

template <int DH, bool BF16, int kInner>
int launch_apply_inner(const Plan& plan, const CUtensorMap& my, const Geo& g, const void* w, void* out, float scale,
                       bool out_by_position, cudaStream_t s)
{
    using SM = SmemA<DH>;
    const size_t smem = (size_t)SM::kW + (size_t)kTileRows * g.ktot * 2;
    if (smem > kMaxDynamicSmem) return -2;
    if (ensure_dynamic_smem((const void*)tc_apply_kernel<DH, BF16, kInner>, kMaxDynamicSmem) != cudaSuccess) {
        cudaGetLastError();
        return -2;
    }
    int ngroups = 1;
    for (int a = 0; a < 3; ++a) ngroups *= plan.p.grp_n[a];
    const dim3 grid((unsigned)(plan.p.ntiles * ngroups), (unsigned)g.Hq, (unsigned)g.B);
    tc_apply_kernel<DH, BF16, kInner><<<grid, kThreads, smem, s>>>(my, plan.p, (const uint16_t*)w, (uint16_t*)out, scale, g.ktot,
                                                         out_by_position ? 1 : 0);
    tc_count_launch();
    const cudaError_t err = cudaGetLastError();
    return err == cudaSuccess ? 0 : (int)err;
}

// ---------------------------------------------------------------------------
// gather kernel:  dst[key] = scale * sum over the (query, head-of-group) pairs that attend to the key of
//                 w[query, slot of the key] * x[query]          (QK backward w.r.t. k: w = dlogits, x = q;
//                                                                 AV backward w.r.t. v: w = attn, x = dout)
// Rows = a box of 128 keys of one (batch, kv head); columns = chunks of 128 queries of the box of queries
// that attend to them (the inverse neighbourhood: a contiguous range per axis, unit
// stride), once per query head of the group.  The threads gather w into a dense 16-bit P^T tile in TMEM
// (lanes of a warp are neighbouring keys, so one load touches one row of w) and acc += P^T X runs on the
// tensor cores with the X chunk staged by TMA and read MN-major.  The order of accumulation is fixed.
// ---------------------------------------------------------------------------
template <int DH>
struct SmemG {
    static constexpr int kHalves = DH / 64;
    static constexpr int kHalf = kTileRows * 128;
    static constexpr int kTile = kHalf * kHalves;
    static constexpr int kX = 0;                          // [kStages] query chunks
    static constexpr int kBar = kX + kStages * kTile;     // barriers, flags: 128 bytes
    static constexpr int kColRow = kBar + 128;            // [2][128] long long: element offset of the column's row of w, -1 = no query
    static constexpr int kColFirst = kColRow + 2048;      // [2][3][128] int: first key of the column's window, per axis
    static constexpr int kTotal = kColFirst + 3072;
    static constexpr uint32_t kColP = 0, kColO = 128, kTmemCols = 256;
};

template <int DH, bool BF16>
__global__ void __launch_bounds__(kThreads, (DH == 64 ? 2 : 1))
tc_gather_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ TcParams P,
                 const uint16_t* __restrict__ w, uint16_t* __restrict__ dst, float scale, int ktot)
{
    using SM = SmemG<DH>;
    constexpr int CH = DH / 2;
    extern __shared__ __align__(1024) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int hk = blockIdx.y, b = blockIdx.z;
    const int quad = warp & 3, team = (warp >> 2) & 1;
    const int prior_abort = *reinterpret_cast<volatile int*>(P.status);

    int rg[3], origin[3], Lp[3], boxlo[3], nc[3];
    if (!cta_geometry(P, blockIdx.x, b, rg, origin, Lp)) return;       // no key of this tile exists
    int nchunks = 1;
#pragma unroll
    for (int a = 0; a < 3; ++a) {
        const int last = origin[a] + P.tile[a] - 1 < Lp[a] - 1 ? origin[a] + P.tile[a] - 1 : Lp[a] - 1;
        int t, hi;
        inverse_range(origin[a], Lp[a], P.K[a], P.causal[a], boxlo[a], t, /*exact=*/false);
        inverse_range(last, Lp[a], P.K[a], P.causal[a], t, hi, /*exact=*/false);
        nc[a] = chunks_along(P, a, hi - boxlo[a] + 1);
        nchunks *= nc[a];
    }
    const int total = nchunks * P.group;

    const uint32_t sbase = smem_u32(smem);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + SM::kBar + 64);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + SM::kBar + 72);
    long long* colrow = reinterpret_cast<long long*>(smem + SM::kColRow);
    const uint32_t bar_x = sbase + SM::kBar + 0;         // [3] X chunk landed
    const uint32_t bar_p = sbase + SM::kBar + 48;        // [2] P^T buffer b stored by every thread
    const uint32_t bar_o = sbase + SM::kBar + 32;        // [2] the MMAs that read P buffer b have finished

    int ld[3] = {0, 0, 0}, ld_head = 0, loaded = 0;
    auto issue_x = [&]() {
        const int s = loaded % kStages;
        const uint32_t bar = bar_x + 8 * s;
        mbar_expect_tx(bar, SM::kTile);
        int X[3];
#pragma unroll
        for (int a = 0; a < 3; ++a) X[a] = rg[a] + P.dil[a] * (boxlo[a] + ld[a] * P.cb[a]);
        const int hx = (hk * P.group + ld_head) * DH;
#pragma unroll
        for (int hf = 0; hf < SM::kHalves; ++hf)
            tma_load_5d(sbase + SM::kX + s * SM::kTile + hf * SM::kHalf, &tmX, bar, hx + 64 * hf, X[2], X[1], X[0], b);
        if (++ld[2] == nc[2]) { ld[2] = 0; if (++ld[1] == nc[1]) { ld[1] = 0; if (++ld[0] == nc[0]) { ld[0] = 0; ++ld_head; } } }
        ++loaded;
    };
    if (warp == 8) {
        if (lane == 0) {
            *abort_flag = ((sbase & 1023u) || prior_abort) ? 1 : 0;
            for (int s = 0; s < kStages; ++s) mbar_init(bar_x + 8 * s, 1);
            mbar_init(bar_p, 256);
            mbar_init(bar_p + 8, 256);
            mbar_init(bar_o, 1);
            mbar_init(bar_o + 8, 1);
            mbar_init_fence();
            fence_async_smem();
            if (!*abort_flag)
                for (int c = 0; c < total && c < kStages; ++c) issue_x();
        }
        __syncwarp();
        tmem_alloc(smem_u32(tmem_slot), SM::kTmemCols);
    }
    // ---- this thread's key ----
    int f[3] = {0, 0, 0}, e[3] = {0, 0, 0}, kx[3] = {0, 0, 0};
    const int row = quad * 32 + lane;
    long long drow = -1;
    int keyslot = 0;
    if (warp < 8) {
        int ri[3];
        row_offsets(P, row, ri);
        bool valid = true;
        long long pflat = 0;
#pragma unroll
        for (int a = 0; a < 3; ++a) {
            kx[a] = origin[a] + ri[a];
            if (kx[a] >= Lp[a]) valid = false;
            pflat = pflat * P.L[a] + (rg[a] + P.dil[a] * kx[a]);
            int qlo, qhi;
            inverse_range(kx[a], Lp[a], P.K[a], P.causal[a], qlo, qhi);
            f[a] = qlo - boxlo[a];
            e[a] = qhi + 1 - boxlo[a];
        }
        if (!valid) { e[0] = f[0]; e[1] = f[1]; e[2] = f[2]; }
        else drow = ((long long)b * P.ltot + pflat) * P.Hkv + hk;
        keyslot = (kx[0] * P.K[1] + kx[1]) * P.K[2] + kx[2];
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 8) {
        // the warp runs the loop converged; the tensor-core instructions execute on an elected lane
        const uint32_t leader = elect_one();
        if (!*abort_flag) {
            constexpr uint32_t idesc = instr_desc(BF16 ? 1 : 0, DH, 0, 1);      // A = P^T from TMEM, B = X MN-major
            bool ok = true;
            for (int c = 0; c < total && ok; ++c) {
                ok = mbar_wait(bar_x + 8 * (c % kStages), (c / kStages) & 1, abort_flag, P.wait_budget) &&
                     mbar_wait(bar_p + 8 * (c & 1), (c >> 1) & 1, abort_flag, P.wait_budget);
                if (!ok) break;
                const uint64_t dx0 = smem_desc(sbase + SM::kX + (c % kStages) * SM::kTile, SM::kHalf, 1024);
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < kChunk / 16; ++ks)
                    mma_ts_e(tmem + SM::kColO, tmem + SM::kColP + 64 * (c & 1) + 8 * ks, dx0 + 128 * ks, idesc, c > 0 || ks > 0, leader);
                mma_commit_e(bar_o + 8 * (c & 1), leader);
                if (c >= 1 && c + 2 < total) {           // the product before this one is done: its X stage is free
                    ok = mbar_wait(bar_o + 8 * ((c - 1) & 1), ((c - 1) >> 1) & 1, abort_flag, P.wait_budget);
                    if (!ok) break;
                    if (leader) issue_x();
                    __syncwarp();
                }
            }
        }
    } else {
        const uint32_t trow = tmem + (static_cast<uint32_t>(quad * 32) << 16);
        const uint16_t* wkey = w + keyslot;
        bool ok = true;
        int ci[3] = {0, 0, 0}, hc = hk * P.group;
        for (int c = 0; c < total; ++c) {
            // ---- per-column tables of this chunk (one thread per column) ----
            // The slot of key kx in the window of query xq is linear in both: (kx - first(xq)) folded over the
            // axes = keyslot(kx) - firstslot(xq).  The table holds, per column, the element offset of the
            // query's row of w minus firstslot; a thread adds its own keyslot.
            long long* crow = colrow + (c & 1) * 128;
            if (tid < 128) {
                const int j[3] = {tid >> (P.cb2_log + P.cb1_log), (tid >> P.cb2_log) & (P.cb[1] - 1), tid & (P.cb[2] - 1)};
                bool inside = true;
                long long pflat = 0;
                int firstslot = 0;
#pragma unroll
                for (int a = 0; a < 3; ++a) {
                    const int xq = boxlo[a] + ci[a] * P.cb[a] + j[a];
                    if (xq < 0 || xq >= Lp[a]) inside = false;
                    pflat = pflat * P.L[a] + (rg[a] + P.dil[a] * xq);
                    const int first = P.causal[a] ? xq - (P.K[a] - 1) : tc_window_start(xq, Lp[a], P.K[a]);
                    firstslot = firstslot * P.K[a] + first;
                }
                crow[tid] = inside ? (((long long)b * P.ltot + pflat) * P.Hq + hc) * ktot - firstslot : 0;
            }
            asm volatile("bar.sync 1, 256;" ::: "memory");
            uint32_t words[2];
#pragma unroll
            for (int pc = 0; pc < 2; ++pc) words[pc] = piece_word(P, ci, 2 * team + pc, f, e);
            if (c >= 2) {                         // P buffer c & 1 was last read by the product of chunk c - 2
                ok = ok && mbar_wait(bar_o + 8 * (c & 1), ((c - 2) >> 1) & 1, abort_flag, P.wait_budget);
                tc_fence_after();
            }
#pragma unroll
            for (int pc = 0; pc < 2; ++pc) {
                uint32_t packed[16];
                if (__any_sync(0xffffffffu, words[pc] != 0u)) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        uint32_t v16[2] = {0u, 0u};
#pragma unroll
                        for (int u = 0; u < 2; ++u) {
                            const int col = 64 * team + 32 * pc + 2 * i + u;
                            if ((words[pc] >> (2 * i + u)) & 1u) v16[u] = wkey[crow[col]];
                        }
                        packed[i] = v16[0] | (v16[1] << 16);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 16; ++i) packed[i] = 0u;
                }
                tmem_st16(trow + SM::kColP + 64 * (c & 1) + 32 * team + 16 * pc, packed);
            }
            tmem_st_wait();
            tc_fence_before();
            mbar_arrive(bar_p + 8 * (c & 1));
            if (++ci[2] == nc[2]) { ci[2] = 0; if (++ci[1] == nc[1]) { ci[1] = 0; if (++ci[0] == nc[0]) { ci[0] = 0; ++hc; } } }
        }
        // ---- every product is in the accumulator: scale, write out this thread's channels ----
        ok = ok && mbar_wait(bar_o + 8 * ((total - 1) & 1), ((total - 1) >> 1) & 1, abort_flag, P.wait_budget);
        tc_fence_after();
#pragma unroll
        for (int part = 0; part < CH / 32; ++part) {
            uint32_t o[32];
            tmem_ld32(trow + SM::kColO + CH * team + 32 * part, o);
            tmem_ld_wait();
            if (drow >= 0 && ok) {
                uint4* o4 = reinterpret_cast<uint4*>(dst + drow * DH + team * CH + 32 * part);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    uint32_t x[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        x[j] = cvt_pack<BF16>(__uint_as_float(o[8 * i + 2 * j]) * scale, __uint_as_float(o[8 * i + 2 * j + 1]) * scale);
                    o4[i] = make_uint4(x[0], x[1], x[2], x[3]);
                }
            }
        }
    }

    if (*abort_flag) abort_grace_sleep();       // loads of a wait that gave up may still be landing
    tc_fence_before();
    __syncthreads();
    if (warp == 8) {
        tc_fence_after();
        tmem_dealloc(tmem, SM::kTmemCols);
        if (lane == 0 && *abort_flag) atomicExch(P.status, 1);
    }
}

template <int DH, bool BF16>
int launch_gather(const Plan& plan, const CUtensorMap& mx, const Geo& g, const void* w, void* dst, float scale,
                  cudaStream_t s)
{
    using SM = SmemG<DH>;
    if (ensure_dynamic_smem((const void*)tc_gather_kernel<DH, BF16>, SM::kTotal) != cudaSuccess) {
        cudaGetLastError();
        return -2;
    }
    int ngroups = 1;
    for (int a = 0; a < 3; ++a) ngroups *= plan.p.grp_n[a];
    const dim3 grid((unsigned)(plan.p.ntiles * ngroups), (unsigned)g.Hkv, (unsigned)g.B);
    tc_gather_kernel<DH, BF16><<<grid, kThreads, SM::kTotal, s>>>(mx, plan.p, (const uint16_t*)w, (uint16_t*)dst, scale, g.ktot);
    tc_count_launch();
    const cudaError_t err = cudaGetLastError();
    return err == cudaSuccess ? 0 : (int)err;
}

} // namespace

// x: the row tensor [B, *L, Hq, D] with strides xs (batch, token, head), indexed by input position;
// y: the key-side tensor [B, *L, Hkv, D] with strides ys.  out: [B, *O, Hq, ktot].
int tc_scores(int dtype, const Geo& g, const void* x, const long long xs[3], const void* y, const long long ys[3],
              float scale, bool neg_inf, void* out, cudaStream_t s, const void* rpb)
{
    int rpb_table = 1;
    if (rpb) {                                   // bias added while the tile is written out: unit stride, no causal axis
        for (int a = 0; a < g.rank; ++a) {
            if (g.st[a] != 1 || g.causal[a] || (g.K[a] & 1) == 0) return -2;
            rpb_table *= 2 * g.K[a] - 1;
        }
        if (g.Hq != g.Hkv) return -2;
    }
    if (dtype != 1 && dtype != 2) return -2;
    if (g.D != 64 && g.D != 128) return -2;
    if (g.extents || g.n_extra) return -2;
    for (int a = 0; a < g.rank; ++a)
        if (!kernel_axis_ok(g, a)) return -2;
    if (xs[2] != g.D || ys[2] != g.D) return -2;
    const long long strs[4] = {xs[0], xs[1], ys[0], ys[1]};
    for (long long st : strs)
        if (st % 8 != 0) return -2;
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15u) return -2;
    if (g.Hq > 65535 || g.B > 65535) return -2;
    // the [128 x slots] tile must fit beside the operand stages (two CTAs per SM at D = 64)
    const size_t budget = g.D == 64 ? 113 * 1024 : 227 * 1024;
    const size_t base = g.D == 64 ? (size_t)SmemS<64>::kOut : (size_t)SmemS<128>::kOut;
    if (base + (size_t)kTileRows * g.ktot * 2 + 16 + (rpb ? 4 * (kTileRows + (size_t)g.ktot) : 0) > budget) return -2;
    Plan plan;
    if (!make_plan(g, plan, kChunk, /*with_stride=*/true)) return -2;
    const bool bf16 = dtype == 2;
    CUtensorMap mx, my;
    if (!encode_map(&mx, x, bf16, plan.p, g.Hq, g.D, xs, plan.box_q, /*query_lattice=*/true) ||
        !encode_map(&my, y, bf16, plan.p, g.Hkv, g.D, ys, plan.box_kv))
        return -2;
    plan.p.status = status_ptr();
    if (!plan.p.status) return -2;
    if (plan.p.work_q == 0) return 0;
    if (g.D == 64)
        return bf16 ? launch_scores<64, true>(plan, mx, my, g, out, scale, neg_inf, s, rpb, rpb_table)
                    : launch_scores<64, false>(plan, mx, my, g, out, scale, neg_inf, s, rpb, rpb_table);
    return bf16 ? launch_scores<128, true>(plan, mx, my, g, out, scale, neg_inf, s, rpb, rpb_table)
                : launch_scores<128, false>(plan, mx, my, g, out, scale, neg_inf, s, rpb, rpb_table);
}

// w: [B, *O, Hq, ktot]; y: [B, *L, Hkv, D] with strides ys; out: [B, *O, Hq, D] (by output row) or, for a
// gradient w.r.t. the queries, [B, *L, Hq, D] by input position (unit stride only).
int tc_apply(int dtype, const Geo& g, const void* w, const void* y, const long long ys[3], float scale,
             bool out_by_position, void* out, cudaStream_t s)
{
    if (dtype != 1 && dtype != 2) return -2;
    if (g.D != 64 && g.D != 128) return -2;
    if (g.extents || g.n_extra) return -2;
    for (int a = 0; a < g.rank; ++a) {
        if (!kernel_axis_ok(g, a)) return -2;
        if (out_by_position && g.st[a] != 1) return -2;
    }
    if (ys[2] != g.D || ys[0] % 8 != 0 || ys[1] % 8 != 0) return -2;
    if ((reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(out)) & 15u) return -2;
    if (g.Hq > 65535 || g.B > 65535) return -2;
    const size_t budget = g.D == 64 ? 113 * 1024 : 227 * 1024;
    const size_t base = g.D == 64 ? (size_t)SmemA<64>::kW : (size_t)SmemA<128>::kW;
    if (base + (size_t)kTileRows * g.ktot * 2 > budget) return -2;
    Plan plan;
    if (!make_plan(g, plan, kChunk, /*with_stride=*/true)) return -2;
    const bool bf16 = dtype == 2;
    CUtensorMap my;
    if (!encode_map(&my, y, bf16, plan.p, g.Hkv, g.D, ys, plan.box_kv)) return -2;
    plan.p.status = status_ptr();
    if (!plan.p.status) return -2;
    if (plan.p.work_q == 0) return 0;
    if (g.D == 64)
        return bf16 ? launch_apply<64, true>(plan, my, g, w, out, scale, out_by_position, s)
                    : launch_apply<64, false>(plan, my, g, w, out, scale, out_by_position, s);
    return bf16 ? launch_apply<128, true>(plan, my, g, w, out, scale, out_by_position, s)
                : launch_apply<128, false>(plan, my, g, w, out, scale, out_by_position, s);
}

// w: [B, *L, Hq, ktot] (unit stride); x: the query-side tensor [B, *L, Hq, D] with strides xs, indexed by
// position; dst: [B, *L, Hkv, D] contiguous.
int tc_gather(int dtype, const Geo& g, const void* w, const void* x, const long long xs[3], float scale,
              void* dst, cudaStream_t s)
{
    if (dtype != 1 && dtype != 2) return -2;
    if (g.D != 64 && g.D != 128) return -2;
    if (g.extents || g.n_extra) return -2;
    for (int a = 0; a < g.rank; ++a)
        if (!kernel_axis_ok(g, a) || g.st[a] != 1) return -2;
    if (xs[2] != g.D || xs[0] % 8 != 0 || xs[1] % 8 != 0) return -2;
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dst)) & 15u) return -2;
    if (g.Hkv > 65535 || g.B > 65535) return -2;
    Plan plan;
    if (!make_plan(g, plan, kChunk)) return -2;
    const bool bf16 = dtype == 2;
    CUtensorMap mx;
    if (!encode_map(&mx, x, bf16, plan.p, g.Hq, g.D, xs, plan.box_kv)) return -2;
    plan.p.status = status_ptr();
    if (!plan.p.status) return -2;
    if (plan.p.work_kv == 0) return 0;
    if (g.D == 64)
        return bf16 ? launch_gather<64, true>(plan, mx, g, w, dst, scale, s) : launch_gather<64, false>(plan, mx, g, w, dst, scale, s);
    return bf16 ? launch_gather<128, true>(plan, mx, g, w, dst, scale, s) : launch_gather<128, false>(plan, mx, g, w, dst, scale, s);
}

} // namespace natten
