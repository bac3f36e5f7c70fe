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

template <int DH, bool BF16>
__global__ void __launch_bounds__(kThreads, (DH == 64 ? 2 : 1))
tc_scores_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmY,
                 const __grid_constant__ TcParams P, uint16_t* __restrict__ out, float scale, uint32_t fill16,
                 int ktot)
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
        if (team == 0) rowout[row] = valid_q ? ((long long)b * P.otot + oflat) * P.Hq + h : -1;
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
        if (lane == 0 && !*abort_flag) {
            constexpr uint32_t idesc = instr_desc(BF16 ? 1 : 0, kChunk, 0, 0);
            const uint64_t dx0 = smem_desc(sbase + SM::kX, 16, 1024);
            auto issue_s = [&](int c) {
                const uint64_t dy0 = smem_desc(sbase + SM::kY + (c % kStages) * SM::kTile, 16, 1024);
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < DH / 16; ++ks) {
                    const uint32_t off = ((ks / 4) * SM::kHalf + (ks % 4) * 32) >> 4;
                    mma_ss(tmem, dx0 + off, dy0 + off, idesc, ks > 0);
                }
                mma_commit(bar_s);
            };
            bool ok = mbar_wait(bar_x, 0, abort_flag) && mbar_wait(bar_y, 0, abort_flag);
            if (ok) issue_s(0);
            for (int c = 0; c < nch && ok; ++c) {
                ok = mbar_wait(bar_s, c & 1, abort_flag);            // the product is done: its Y stage is free
                if (!ok) break;
                if (c + kStages < nch) issue_y();
                ok = mbar_wait(bar_sp, c & 1, abort_flag);           // S(c) read by every thread
                if (!ok) break;
                if (c + 1 < nch) {
                    ok = mbar_wait(bar_y + 8 * ((c + 1) % kStages), ((c + 1) / kStages) & 1, abort_flag);
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
            ok = ok && mbar_wait(bar_s, c & 1, abort_flag);
            tc_fence_after();
#pragma unroll
            for (int pc = 0; pc < 2; ++pc) {
                if (!__any_sync(0xffffffffu, words[pc] != 0u)) continue;
                uint32_t s[32];
                tmem_ld32(trow + 64 * team + 32 * pc, s);
                tmem_ld_wait();
                if (ok) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        if ((words[pc] >> i) & 1u) {
                            const float v = __uint_as_float(s[i]) * scale;
                            uint16_t bits;
                            if (BF16) { const __nv_bfloat16 t = __float2bfloat16_rn(v); bits = *reinterpret_cast<const uint16_t*>(&t); }
                            else { const __half t = __float2half_rn(v); bits = *reinterpret_cast<const uint16_t*>(&t); }
                            myrow[base + colslot[64 * team + 32 * pc + i]] = bits;
                        }
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
            int r = tid / ktot, j = tid - r * ktot;
            const int total = kTileRows * ktot;
            for (int idx = tid; idx < total; idx += 256) {
                const long long orow = rowout[r];
                if (orow >= 0) out[orow * ktot + j] = tile[idx];
                j += 256;
                while (j >= ktot) { j -= ktot; ++r; }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 8) {
        tc_fence_after();
        tmem_dealloc(tmem, 128);
        if (lane == 0 && *abort_flag) atomicExch(P.status, 1);
    }
}

template <int DH, bool BF16>
int launch_scores(const Plan& plan, const CUtensorMap& mx, const CUtensorMap& my, const Geo& g, void* out,
                  float scale, bool neg_inf, cudaStream_t s)
{
    using SM = SmemS<DH>;
    const size_t smem = (size_t)SM::kOut + (size_t)kTileRows * g.ktot * 2;
    static size_t attr = 0;
    if (smem > attr) {
        if (cudaFuncSetAttribute(tc_scores_kernel<DH, BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
            cudaGetLastError();
            return -2;
        }
        attr = smem;
    }
    int ngroups = 1;
    for (int a = 0; a < 3; ++a) ngroups *= plan.p.grp_n[a];
    const dim3 grid((unsigned)(plan.p.ntiles * ngroups), (unsigned)g.Hq, (unsigned)g.B);
    const uint32_t fill = neg_inf ? (BF16 ? 0xFF80u : 0xFC00u) : 0u;
    tc_scores_kernel<DH, BF16><<<grid, kThreads, smem, s>>>(mx, my, plan.p, (uint16_t*)out, scale, fill, g.ktot);
    tc_count_launch();
    const cudaError_t err = cudaGetLastError();
    return err == cudaSuccess ? 0 : (int)err;
}

} // namespace

// x: the row tensor [B, *L, Hq, D] with strides xs (batch, token, head), indexed by input position;
// y: the key-side tensor [B, *L, Hkv, D] with strides ys.  out: [B, *O, Hq, ktot].
int tc_scores(int dtype, const Geo& g, const void* x, const long long xs[3], const void* y, const long long ys[3],
              float scale, bool neg_inf, void* out, cudaStream_t s)
{
    if (dtype != 1 && dtype != 2) return -2;
    if (g.D != 64 && g.D != 128) return -2;
    if (g.extents || g.n_extra) return -2;
    for (int a = 0; a < g.rank; ++a)
        if ((g.K[a] & 1) == 0) return -2;
    if (xs[2] != g.D || ys[2] != g.D) return -2;
    const long long strs[4] = {xs[0], xs[1], ys[0], ys[1]};
    for (long long st : strs)
        if (st % 8 != 0) return -2;
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15u) return -2;
    if (g.Hq > 65535 || g.B > 65535) return -2;
    // the [128 x slots] tile must fit beside the operand stages (two CTAs per SM at D = 64)
    const size_t budget = g.D == 64 ? 113 * 1024 : 227 * 1024;
    const size_t base = g.D == 64 ? (size_t)SmemS<64>::kOut : (size_t)SmemS<128>::kOut;
    if (base + (size_t)kTileRows * g.ktot * 2 > budget) return -2;
    Plan plan;
    if (!make_plan(g, plan, kChunk, /*with_stride=*/true)) return -2;
    const bool bf16 = dtype == 2;
    CUtensorMap mx, my;
    if (!encode_map(&mx, x, bf16, plan.p, g.Hq, g.D, xs, plan.box_q, /*query_lattice=*/true) ||
        !encode_map(&my, y, bf16, plan.p, g.Hkv, g.D, ys, plan.box_kv))
        return -2;
    plan.p.status = status_ptr();
    plan.p.trace = nullptr;
    if (!plan.p.status) return -2;
    if (plan.p.work_q == 0) return 0;
    if (g.D == 64)
        return bf16 ? launch_scores<64, true>(plan, mx, my, g, out, scale, neg_inf, s)
                    : launch_scores<64, false>(plan, mx, my, g, out, scale, neg_inf, s);
    return bf16 ? launch_scores<128, true>(plan, mx, my, g, out, scale, neg_inf, s)
                : launch_scores<128, false>(plan, mx, my, g, out, scale, neg_inf, s);
}

} // namespace natten
