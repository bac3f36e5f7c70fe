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

constexpr int kStages = 3;
constexpr int kThreads = 160;            // 4 softmax warps + 1 TMA/MMA warp
constexpr uint32_t kTmemCols = 256;
constexpr uint32_t kColS = 0, kColP = 128, kColO = 192;

// Shared-memory map (dynamic, base must be 1024-byte aligned).
template <int DH>
struct SmemMap {
    static constexpr int kHalves = DH / 64;
    static constexpr int kTile = kTileRows * 128 * kHalves;       // bytes of one [128 x DH] 16-bit tile
    static constexpr int kQ = 0;
    static constexpr int kK = kQ + kTile;
    static constexpr int kV = kK + kStages * kTile;
    static constexpr int kBar = kV + kStages * kTile;
    // barriers: q, kv_full[3], s_full, sp_ready, o_full  (8 bytes each) + tmem ptr + abort flag
    static constexpr int kTotal = kBar + 128;
};

__device__ __forceinline__ int tc_window_start(int p, int L, int K) { return window_start(p, L, K, 1); }

template <int DH, bool BF16>
__global__ void __launch_bounds__(kThreads, (DH == 64 ? 2 : 1))
tc_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
              const __grid_constant__ CUtensorMap tmV, const __grid_constant__ TcParams P,
              uint16_t* __restrict__ out, float* __restrict__ lse)
{
    using SM = SmemMap<DH>;
    extern __shared__ __align__(1024) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = blockIdx.y, b = blockIdx.z, hk = h / P.group;

    // ---- CTA geometry -------------------------------------------------------
    int gidx = blockIdx.x / P.ntiles, tidx = blockIdx.x % P.ntiles;
    int rg[3], origin[3], Ls[3], Lp[3], lo[3];
    bool cta_active = true;
    for (int a = 2; a >= 0; --a) {
        rg[a] = gidx % P.dil[a]; gidx /= P.dil[a];
        origin[a] = (tidx % P.ntile[a]) * P.tile[a]; tidx /= P.ntile[a];
        const int ea = a - (3 - P.rank);
        Ls[a] = (P.extents && ea >= 0) ? P.extents[b * P.rank + ea] : P.L[a];
        Lp[a] = rg[a] < Ls[a] ? (Ls[a] - rg[a] + P.dil[a] - 1) / P.dil[a] : 0;
        if (origin[a] >= Lp[a]) cta_active = false;
        lo[a] = P.causal[a] ? origin[a] - (P.K[a] - 1) : tc_window_start(origin[a], Lp[a] > 0 ? Lp[a] : 1, P.K[a]);
    }

    // ---- per-thread query row (softmax warps) -------------------------------
    int f[3] = {0, 0, 0}, e[3] = {0, 0, 0};
    bool valid_q = false, in_tensor = false;
    long long out_row = 0;
    if (warp < 4) {
        int r = tid, pflat_ok = 1;
        int qi[3], pa[3];
        qi[2] = r % P.tile[2]; r /= P.tile[2];
        qi[1] = r % P.tile[1]; r /= P.tile[1];
        qi[0] = r;
        valid_q = true; in_tensor = true;
        long long pflat = 0;
        for (int a = 0; a < 3; ++a) {
            const int qa = origin[a] + qi[a];
            pa[a] = rg[a] + P.dil[a] * qa;
            if (qa >= Lp[a]) valid_q = false;
            if (pa[a] >= P.L[a]) in_tensor = false;
            pflat = pflat * P.L[a] + pa[a];
            if (cta_active) {
                const int first = P.causal[a] ? qa - (P.K[a] - 1) : tc_window_start(qa, Lp[a], P.K[a]);
                const int fa = first > 0 ? first : 0;
                const int la = first + P.K[a] < Lp[a] ? first + P.K[a] : Lp[a];
                f[a] = fa - lo[a];
                e[a] = la - lo[a];
            }
        }
        (void)pflat_ok;
        if (!valid_q) { e[0] = f[0]; e[1] = f[1]; e[2] = f[2]; }
        out_row = (((long long)b * P.ltot + pflat) * P.Hq + h);
    }

    if (!cta_active) {                       // nothing to attend: padding rows are zero
        if (warp < 4 && in_tensor) {
            uint4* o4 = reinterpret_cast<uint4*>(out + out_row * DH);
#pragma unroll
            for (int i = 0; i < DH / 8; ++i) o4[i] = make_uint4(0, 0, 0, 0);
            lse[out_row] = 0.f;
        }
        return;
    }

    // ---- shared memory, barriers, TMEM --------------------------------------
    const uint32_t sbase = smem_u32(smem);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + SM::kBar + 64);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + SM::kBar + 72);
    const uint32_t bar_q = sbase + SM::kBar + 0;
    const uint32_t bar_kv = sbase + SM::kBar + 8;       // [3]
    const uint32_t bar_s = sbase + SM::kBar + 32;
    const uint32_t bar_sp = sbase + SM::kBar + 40;
    const uint32_t bar_o = sbase + SM::kBar + 48;

    if (tid == 0) {
        // swizzled tiles need a 1024-byte aligned base; once any CTA has given up, the rest bail out
        *abort_flag = ((sbase & 1023u) || *reinterpret_cast<volatile int*>(P.status)) ? 1 : 0;
        mbar_init(bar_q, 1);
        for (int s = 0; s < kStages; ++s) mbar_init(bar_kv + 8 * s, 1);
        mbar_init(bar_s, 1);
        mbar_init(bar_sp, 128);
        mbar_init(bar_o, 1);
        mbar_init_fence();
    }
    if (warp == 4) {
        tmem_alloc(smem_u32(tmem_slot), kTmemCols);
        if (lane == 0) { tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV); }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const int nch = P.nchunks;

    if (warp == 4) {
        // =====================================================================
        // TMA + MMA issue (one thread)
        // =====================================================================
        if (lane == 0 && !*abort_flag) {
            auto issue_kv = [&](int c) {
                int cc = c, ci[3];
                ci[2] = cc % P.nchunk[2]; cc /= P.nchunk[2];
                ci[1] = cc % P.nchunk[1]; cc /= P.nchunk[1];
                ci[0] = cc;
                int X[3];
                for (int a = 0; a < 3; ++a) X[a] = rg[a] + P.dil[a] * (lo[a] + ci[a] * P.cb[a]);
                const int s = c % kStages;
                const uint32_t bar = bar_kv + 8 * s;
                mbar_expect_tx(bar, 2 * SM::kTile);
                for (int hf = 0; hf < SM::kHalves; ++hf) {
                    tma_load_5d(sbase + SM::kK + s * SM::kTile + hf * (kChunk * 128), &tmK, bar,
                                hk * DH + 64 * hf, X[2], X[1], X[0], b);
                    tma_load_5d(sbase + SM::kV + s * SM::kTile + hf * (kChunk * 128), &tmV, bar,
                                hk * DH + 64 * hf, X[2], X[1], X[0], b);
                }
            };
            mbar_expect_tx(bar_q, SM::kTile);
            for (int hf = 0; hf < SM::kHalves; ++hf)
                tma_load_5d(sbase + SM::kQ + hf * (kTileRows * 128), &tmQ, bar_q, h * DH + 64 * hf,
                            rg[2] + P.dil[2] * origin[2], rg[1] + P.dil[1] * origin[1],
                            rg[0] + P.dil[0] * origin[0], b);
            for (int c = 0; c < nch && c < kStages; ++c) issue_kv(c);

            constexpr uint32_t idesc_qk = instr_desc(BF16 ? 1 : 0, kChunk, 0, 0);
            constexpr uint32_t idesc_pv = instr_desc(BF16 ? 1 : 0, DH, 0, 1);
            auto issue_qk = [&](int c) {
                const int s = c % kStages;
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < DH / 16; ++ks) {
                    const uint32_t off = (ks / 4) * (kTileRows * 128) + (ks % 4) * 32;
                    mma_ss(tmem + kColS, smem_desc(sbase + SM::kQ + off, 16, 1024),
                           smem_desc(sbase + SM::kK + s * SM::kTile + off, 16, 1024), idesc_qk, ks > 0);
                }
                mma_commit(bar_s);
            };
            auto issue_pv = [&](int c) {
                const int s = c % kStages;
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < kChunk / 16; ++ks)
                    mma_ts(tmem + kColO, tmem + kColP + 8 * ks,
                           smem_desc(sbase + SM::kV + s * SM::kTile + ks * 2048, kChunk * 128, 1024),
                           idesc_pv, ks > 0);
                mma_commit(bar_o);
            };

            bool ok = mbar_wait(bar_q, 0, abort_flag);
            for (int c = 0; c < nch && ok; ++c) {
                if (c == 0) {
                    ok = mbar_wait(bar_kv, 0, abort_flag);
                    if (ok) issue_qk(0);
                }
                ok = ok && mbar_wait(bar_sp, c & 1, abort_flag);     // S(c) consumed, P(c) stored
                if (!ok) break;
                issue_pv(c);
                if (c + 1 < nch) {
                    ok = mbar_wait(bar_kv + 8 * ((c + 1) % kStages), ((c + 1) / kStages) & 1, abort_flag);
                    if (!ok) break;
                    issue_qk(c + 1);
                }
                if (c + kStages < nch) {
                    ok = mbar_wait(bar_o, c & 1, abort_flag);        // stage c % kStages is free again
                    if (!ok) break;
                    issue_kv(c + kStages);
                }
            }
        }
    } else {
        // =====================================================================
        // softmax warps: thread = query row
        // =====================================================================
        const uint32_t trow = tmem + (static_cast<uint32_t>(warp * 32) << 16);
        float m = -INFINITY, l = 0.f;
        float acc[DH];
#pragma unroll
        for (int i = 0; i < DH; ++i) acc[i] = 0.f;
        const int seg = P.cb[2] < 32 ? P.cb[2] : 32;
        const int nseg = 32 / seg;
        bool ok = true;

        for (int c = 0; c < nch; ++c) {
            // ---- validity words of this chunk (bit j of word pc <-> column 32*pc + j) ----
            int cc = c, ci[3];
            ci[2] = cc % P.nchunk[2]; cc /= P.nchunk[2];
            ci[1] = cc % P.nchunk[1]; cc /= P.nchunk[1];
            ci[0] = cc;
            uint32_t words[4];
#pragma unroll
            for (int pc = 0; pc < 4; ++pc) {
                uint32_t w = 0;
                for (int sg = 0; sg < nseg; ++sg) {
                    const int jj = 32 * pc + sg * seg;
                    const int j2 = jj & (P.cb[2] - 1);
                    const int j1 = (jj >> P.cb2_log) & (P.cb[1] - 1);
                    const int j0 = jj >> (P.cb2_log + P.cb1_log);
                    const int i0 = ci[0] * P.cb[0] + j0, i1 = ci[1] * P.cb[1] + j1;
                    const int base2 = ci[2] * P.cb[2] + j2;
                    int lo2 = f[2] - base2, hi2 = e[2] - base2;
                    lo2 = lo2 > 0 ? lo2 : 0;
                    hi2 = hi2 < seg ? hi2 : seg;
                    if (i0 >= f[0] && i0 < e[0] && i1 >= f[1] && i1 < e[1] && hi2 > lo2) {
                        const uint32_t run = (hi2 - lo2 >= 32) ? 0xffffffffu : ((1u << (hi2 - lo2)) - 1u);
                        w |= (run << lo2) << (sg * seg);
                    }
                }
                words[pc] = w;
            }

            ok = ok && mbar_wait(bar_s, c & 1, abort_flag);
            tc_fence_after();

            // ---- pass 1: row maximum over the valid columns ----
            float mc = -INFINITY;
#pragma unroll
            for (int pc = 0; pc < 4; ++pc) {
                if (!__any_sync(0xffffffffu, words[pc] != 0u)) continue;
                uint32_t s[32];
                tmem_ld32(trow + kColS + 32 * pc, s);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    mc = fmaxf(mc, ((words[pc] >> i) & 1u) ? __uint_as_float(s[i]) : -INFINITY);
            }
            if (!ok) mc = -INFINITY;
            const float m_new = fmaxf(m, mc);
            const float alpha = (m == -INFINITY) ? 0.f : fast_exp2((m - m_new) * P.scale_log2);
            const float mb = (m_new == -INFINITY) ? 0.f : m_new * P.scale_log2;

            // ---- fold the previous chunk's P V into the accumulators ----
            if (c > 0) {
                ok = ok && mbar_wait(bar_o, (c - 1) & 1, abort_flag);
                tc_fence_after();
#pragma unroll
                for (int part = 0; part < DH / 32; ++part) {
                    uint32_t o[32];
                    tmem_ld32(trow + kColO + 32 * part, o);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        acc[32 * part + i] = (acc[32 * part + i] + __uint_as_float(o[i])) * alpha;
                }
            }

            // ---- pass 2: probabilities -> TMEM (16-bit pairs), row sum ----
            float rowsum = 0.f;
#pragma unroll
            for (int pc = 0; pc < 4; ++pc) {
                uint32_t packed[16];
                if (__any_sync(0xffffffffu, words[pc] != 0u)) {
                    uint32_t s[32];
                    tmem_ld32(trow + kColS + 32 * pc, s);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const float p0 = ((words[pc] >> (2 * i)) & 1u)
                                             ? fast_exp2(__uint_as_float(s[2 * i]) * P.scale_log2 - mb) : 0.f;
                        const float p1 = ((words[pc] >> (2 * i + 1)) & 1u)
                                             ? fast_exp2(__uint_as_float(s[2 * i + 1]) * P.scale_log2 - mb) : 0.f;
                        rowsum += p0 + p1;
                        if (BF16) {
                            __nv_bfloat162 t = __floats2bfloat162_rn(p0, p1);
                            packed[i] = *reinterpret_cast<uint32_t*>(&t);
                        } else {
                            __half2 t = __floats2half2_rn(p0, p1);
                            packed[i] = *reinterpret_cast<uint32_t*>(&t);
                        }
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 16; ++i) packed[i] = 0u;
                }
                tmem_st16(trow + kColP + 16 * pc, packed);
            }
            if (!ok) rowsum = 0.f;
            l = l * alpha + rowsum;
            m = m_new;
            tmem_st_wait();
            tc_fence_before();
            mbar_arrive(bar_sp);
        }

        // ---- last chunk's P V, normalise, write out ----
        ok = ok && mbar_wait(bar_o, (nch - 1) & 1, abort_flag);
        tc_fence_after();
#pragma unroll
        for (int part = 0; part < DH / 32; ++part) {
            uint32_t o[32];
            tmem_ld32(trow + kColO + 32 * part, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) acc[32 * part + i] += __uint_as_float(o[i]);
        }
        if (in_tensor) {
            const bool live = valid_q && l > 0.f && ok;
            const float inv = live ? 1.f / l : 0.f;
            uint4* o4 = reinterpret_cast<uint4*>(out + out_row * DH);
#pragma unroll
            for (int i = 0; i < DH / 8; ++i) {
                uint32_t w[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float a0 = live ? acc[8 * i + 2 * j] * inv : 0.f;
                    const float a1 = live ? acc[8 * i + 2 * j + 1] * inv : 0.f;
                    if (BF16) {
                        __nv_bfloat162 t = __floats2bfloat162_rn(a0, a1);
                        w[j] = *reinterpret_cast<uint32_t*>(&t);
                    } else {
                        __half2 t = __floats2half2_rn(a0, a1);
                        w[j] = *reinterpret_cast<uint32_t*>(&t);
                    }
                }
                o4[i] = make_uint4(w[0], w[1], w[2], w[3]);
            }
            // natural-log lse of scale * logits
            lse[out_row] = live ? (m * P.scale_log2 + log2f(l)) * 0.6931471805599453f : 0.f;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 4) {
        tc_fence_after();
        tmem_dealloc(tmem, kTmemCols);
        if (lane == 0 && *abort_flag) atomicExch(P.status, 1);
    }
}

} // namespace

int tc_fused_fwd(int dtype, const Geo& g, const void* q, const void* k, const void* v, const void* ek,
                 const void* ev, void* out, void* lse, cudaStream_t s)
{
    (void)ek; (void)ev;
    if (!tc_eligible(dtype, g, q, k, v)) return -2;
    Plan plan;
    if (!make_plan(g, plan)) return -2;
    const bool bf16 = dtype == 2;
    CUtensorMap mq, mk, mv;
    if (!encode_map(&mq, q, bf16, plan.p, g.Hq, g.D, g.qs, plan.box_q) ||
        !encode_map(&mk, k, bf16, plan.p, g.Hkv, g.D, g.ks, plan.box_kv) ||
        !encode_map(&mv, v, bf16, plan.p, g.Hkv, g.Dv, g.vs, plan.box_kv))
        return -2;
    plan.p.status = status_ptr();
    plan.p.trace = trace_ptr();
    if (!plan.p.status) return -2;
    int ngroups = 1;
    for (int a = 0; a < 3; ++a) ngroups *= plan.p.dil[a];
    const dim3 grid((unsigned)(plan.p.ntiles * ngroups), (unsigned)g.Hq, (unsigned)g.B);
    if (grid.x == 0 || g.B == 0) return 0;
    if (g.Hq > 65535 || g.B > 65535) return -2;
    using SM = SmemMap<64>;
    cudaError_t err;
    if (bf16) {
        static bool once = false;
        if (!once) { cudaFuncSetAttribute(tc_fwd_kernel<64, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::kTotal); once = true; }
        tc_fwd_kernel<64, true><<<grid, kThreads, SM::kTotal, s>>>(mq, mk, mv, plan.p, (uint16_t*)out, (float*)lse);
    } else {
        static bool once = false;
        if (!once) { cudaFuncSetAttribute(tc_fwd_kernel<64, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::kTotal); once = true; }
        tc_fwd_kernel<64, false><<<grid, kThreads, SM::kTotal, s>>>(mq, mk, mv, plan.p, (uint16_t*)out, (float*)lse);
    }
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
