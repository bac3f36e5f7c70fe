// Shared by the tensor-core kernels: launch geometry (tile / chunk shapes), tensor-map
// encoding, eligibility and the per-row mask words.
#pragma once
#include "device_cache.cuh"
#include "geometry.cuh"
#include "tc_common.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <mutex>

namespace natten {
namespace tcplan {

using namespace tc;
using natten::ensure_dynamic_smem;
using natten::sm_count;

constexpr int kTileRows = 128;           // rows per CTA     (MMA M)
constexpr int kChunk = 128;              // columns per chunk (MMA N of S, K of the second MMA)

// Geometry is always three axes; lower ranks get leading axes of extent 1.
struct TcParams {
    int L[3], K[3], dil[3], causal[3];
    int tile[3], cb[3], nchunk[3], ntile[3];
    int cb0_log, cb1_log, cb2_log;
    int tile1_log, tile2_log;            // tile extents are powers of two
    unsigned ntile_mul[3], dil_mul[3];   // ceil(2^32 / d) for d >= 2, 0 for d == 1 (see fast_div)
    int rank, B, Hq, Hkv, group, ntiles, nchunks;
    int n_extra;           // additional key/value tokens every query attends to (0 = none)
    int ngroups;           // dilation sub-grids = prod(dil)
    unsigned per_head;     // tiles of one (batch, head) = ntiles * ngroups
    unsigned work_q, work_kv;   // work items of a launch: per_head * B * Hq / Hkv
    float scale_log2, scale;
    const int* extents;
    long long ltot;
    int* status;
    // Interleaved chunks (forward only): along an axis with il > 1 chunk ci holds the box columns
    // ci, ci + il, ci + 2*il, ... instead of a contiguous block, so that every chunk carries a share of
    // every row's window.  il == 1: blocked (chunk ci = columns [ci*cb, (ci+1)*cb)).
    int il[3];
    unsigned il_mul[3], group_mul;       // fast_div multipliers of il[] and of the GQA group size
    // Head dims other than 64 / 128 run on the next larger kernel with zero-padded channels: the tensor
    // maps then carry the head as an axis of its own ([D, H, X2, X1, B]; ranks 1 and 2) and a 64-channel
    // box reads zeros past the real head dim `dreal`.  Outputs are written `dreal` channels wide.
    int dreal, split_heads;
    long long wait_budget; // cycles a barrier wait may take before the CTA gives up
    int inject;            // test hook: 1 = the forward's first query barrier expects bytes that never arrive
    // Output stride (forward only).  Inside dilation group r of an axis the queries sit at the
    // sub-grid indices x = qx0[axis][r] + qstep[axis] * i, i = 0, 1, ... (qx0 < 0: the group holds no
    // query); with stride 1 that is every index.  Output position = input position / st.
    int st[3], qstep[3], O[3];
    int qx0[3][8];
    // Dilation groups that hold queries: r = grp_step * j, j < grp_n (every group when the stride is 1).
    int grp_n[3], grp_step[3];
    unsigned grp_mul[3];
    long long otot;
};

int* status_ptr();   // device address of the library's status word on the current device (tc_status.cu)
long long debug_wait_budget();   // barrier-wait budget in cycles (test hook; default kWaitBudgetCycles)
int debug_inject();              // test hook, see TcParams::inject

// n / d with a precomputed multiplier; exact while n * d < 2^32 (checked on the host).
__device__ __forceinline__ unsigned fast_div(unsigned n, unsigned mul) { return mul ? __umulhi(n, mul) : n; }

// Block index -> dilation residues rg, tile origin, sub-grid extents Lp (innermost axis fastest,
// dilation group slowest); returns whether the tile holds any row of this sample.
__device__ __forceinline__ bool cta_geometry(const TcParams& P, unsigned bx, int b, int (&rg)[3],
                                             int (&origin)[3], int (&Lp)[3])
{
    unsigned x = bx;
#pragma unroll
    for (int a = 2; a >= 0; --a) {
        const unsigned q = fast_div(x, P.ntile_mul[a]);
        origin[a] = static_cast<int>(x - q * P.ntile[a]) * P.tile[a];
        x = q;
    }
    bool active = true;
#pragma unroll
    for (int a = 2; a >= 0; --a) {
        const unsigned q = fast_div(x, P.grp_mul[a]);
        rg[a] = static_cast<int>(x - q * P.grp_n[a]) * P.grp_step[a];
        x = q;
        const int ea = a - (3 - P.rank);
        const int Ls = (P.extents && ea >= 0) ? P.extents[b * P.rank + ea] : P.L[a];
        Lp[a] = rg[a] < Ls ? static_cast<int>(fast_div(Ls - rg[a] + P.dil[a] - 1, P.dil_mul[a])) : 0;
        if (origin[a] >= Lp[a]) active = false;
    }
    return active;
}

// Tile load whose first coordinate is head * dh + channel block: with a head axis of its own in the map
// (split_heads) the two are separated again.  dh is the kernel's (padded) head dim, a power of two.
__device__ __forceinline__ void tma_load_heads(uint32_t dst, const CUtensorMap* map, uint32_t bar, const TcParams& P,
                                               int dh, int c0, int c1, int c2, int c3, int c4)
{
    if (P.split_heads) tma_load_5d(dst, map, bar, c0 & (dh - 1), c0 / dh, c1, c2, c4);
    else tma_load_5d(dst, map, bar, c0, c1, c2, c3, c4);
}
__device__ __forceinline__ void tma_store_heads(const CUtensorMap* map, uint32_t src, const TcParams& P, int dh, int c0,
                                                int c1, int c2, int c3, int c4)
{
    if (P.split_heads) tma_store_5d(map, src, c0 & (dh - 1), c0 / dh, c1, c2, c4);
    else tma_store_5d(map, src, c0, c1, c2, c3, c4);
}

// Chunks needed to cover `extent` columns along axis a (chunk extents are powers of two).
__device__ __forceinline__ int chunks_along(const TcParams& P, int a, int extent)
{
    if (P.il[a] > 1) return extent < P.il[a] ? extent : P.il[a];      // interleaved: chunk ci starts at column ci
    const int lg = a == 0 ? P.cb0_log : (a == 1 ? P.cb1_log : P.cb2_log);
    return (extent + P.cb[a] - 1) >> lg;
}

// Queries x of a sub-grid of length L whose window holds key n, as the range [qlo, qhi].  The window
// start s(x) = window_start(x, L, K, 1) never decreases with x, so the set is a range.  Every window
// that is clamped at the end starts at `last`: L-K for an odd kernel, L-K-1 for an even one (the
// reference's window arithmetic never reaches the last key with an even kernel).  `exact` = false
// gives a range that is never empty (a superset, for bounding boxes); with `exact` a key that no query
// attends to gets qhi < qlo.
__device__ __forceinline__ void inverse_range(int n, int L, int K, int causal, int& qlo, int& qhi, bool exact = true)
{
    if (causal) {
        qlo = n;
        qhi = n + K - 1 < L - 1 ? n + K - 1 : L - 1;
        return;
    }
    const int nh = K / 2, last = L - K - 1 + (K & 1);
    qlo = (n <= K - 1) ? 0 : n - (K - 1 - nh);
    qhi = (n >= last) ? L - 1 : n + nh;
    if (exact && n > last + K - 1) qhi = qlo - 1;
}

// Row r (0..127) of the tile -> offsets along the three axes.
__device__ __forceinline__ void row_offsets(const TcParams& P, int r, int (&ri)[3])
{
    ri[2] = r & (P.tile[2] - 1);
    ri[1] = (r >> P.tile2_log) & (P.tile[1] - 1);
    ri[0] = r >> (P.tile2_log + P.tile1_log);
}

__device__ __forceinline__ float fast_exp2(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Validity bits of one 32-column piece of a chunk for a row whose valid columns are the
// box [f0,e0) x [f1,e1) x [f2,e2) (box coordinates).  ci = chunk index per axis,
// bit j <-> column 32*pc + j of the chunk; columns run (j0, j1, j2) row-major over cb.
__device__ __forceinline__ uint32_t piece_word(const TcParams& P, const int (&ci)[3], int pc,
                                               const int (&f)[3], const int (&e)[3])
{
    const int seg = P.cb[2] < 32 ? P.cb[2] : 32;
    const int nseg = 32 / seg;
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
    return w;
}

// Per-sample extents: a column chunk may reach past the sample's extent into rows that exist in
// memory (padding up to the tensor's extent) but do not belong to the sample.  The reference never
// reads them (it slices each sample, src/natten_mps/_core/pure.py:586-599); here their
// probabilities are zero, but a zero times a non-finite padding value would still poison the
// accumulating product, so those rows of the staged tiles are overwritten with zeros before the
// tensor cores read them.  Called by one thread; box0[] = sub-grid coordinate of the chunk's
// first column per axis; `tiles` = the two [cols x 64*halves] tiles of the stage.
__device__ __forceinline__ void zero_rows_past_extent(const TcParams& P, const int (&box0)[3], const int (&Lp)[3],
                                                      int cols, int halves, int half_bytes,
                                                      uint8_t* tile1, uint8_t* tile2)
{
    // box0[] is the coordinate of column 0; successive columns are il apart (1 when blocked)
    bool crosses = false;
#pragma unroll
    for (int a = 0; a < 3; ++a) crosses = crosses || (box0[a] + (P.cb[a] - 1) * P.il[a] + 1 > Lp[a]);
    if (!crosses) return;
    for (int j = 0; j < cols; ++j) {
        const int j2 = j & (P.cb[2] - 1);
        const int j1 = (j >> P.cb2_log) & (P.cb[1] - 1);
        const int j0 = j >> (P.cb2_log + P.cb1_log);
        if (box0[0] + j0 * P.il[0] < Lp[0] && box0[1] + j1 * P.il[1] < Lp[1] && box0[2] + j2 * P.il[2] < Lp[2]) continue;
        for (int hf = 0; hf < halves; ++hf) {
            uint4* r1 = reinterpret_cast<uint4*>(tile1 + hf * half_bytes + j * 128);
            uint4* r2 = reinterpret_cast<uint4*>(tile2 + hf * half_bytes + j * 128);
#pragma unroll
            for (int i = 0; i < 8; ++i) { r1[i] = make_uint4(0, 0, 0, 0); r2[i] = make_uint4(0, 0, 0, 0); }
        }
    }
    fence_async_smem();          // the tensor cores read shared memory through the async proxy
}

// Columns j of chunk ci (along axis a) that fall inside the box range [f, e): j in [jl, jh), clamped to the chunk.
__device__ __forceinline__ void chunk_range(const TcParams& P, int a, int ci, int f, int e, int& jl, int& jh)
{
    if (P.il[a] == 1) {
        jl = f - ci * P.cb[a];
        jh = e - ci * P.cb[a];
    } else {                                     // column j sits at box coordinate ci + il * j
        const int x = f - ci + P.il[a] - 1, y = e - ci + P.il[a] - 1;
        jl = x > 0 ? (int)fast_div((unsigned)x, P.il_mul[a]) : 0;
        jh = y > 0 ? (int)fast_div((unsigned)y, P.il_mul[a]) : 0;
    }
    jl = jl > 0 ? jl : 0;
    jh = jh < P.cb[a] ? jh : P.cb[a];
}

// Box coordinate (relative to the box origin) of column j of chunk ci along axis a.
__device__ __forceinline__ int chunk_coord(const TcParams& P, int a, int ci, int j)
{
    return P.il[a] == 1 ? ci * P.cb[a] + j : ci + P.il[a] * j;
}

// Validity bits of one 32-column piece from per-axis column ranges [jl, jh) (see chunk_range).
__device__ __forceinline__ uint32_t piece_word_ranges(const TcParams& P, int pc, const int (&jl)[3], const int (&jh)[3])
{
    const int seg = P.cb[2] < 32 ? P.cb[2] : 32;
    const int nseg = 32 / seg;
    uint32_t w = 0;
    for (int sg = 0; sg < nseg; ++sg) {
        const int jj = 32 * pc + sg * seg;
        const int j2 = jj & (P.cb[2] - 1);
        const int j1 = (jj >> P.cb2_log) & (P.cb[1] - 1);
        const int j0 = jj >> (P.cb2_log + P.cb1_log);
        int lo2 = jl[2] - j2, hi2 = jh[2] - j2;
        lo2 = lo2 > 0 ? lo2 : 0;
        hi2 = hi2 < seg ? hi2 : seg;
        if (j0 >= jl[0] && j0 < jh[0] && j1 >= jl[1] && j1 < jh[1] && hi2 > lo2) {
            const uint32_t run = (hi2 - lo2 >= 32) ? 0xffffffffu : ((1u << (hi2 - lo2)) - 1u);
            w |= (run << lo2) << (sg * seg);
        }
    }
    return w;
}

// Packed 16-bit pair arithmetic (element 0 in the low half).
template <bool BF16> __device__ __forceinline__ uint32_t cvt_pack(float lo, float hi)
{
    uint32_t d;
    if (BF16) asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    else asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    return d;
}
template <bool BF16> __device__ __forceinline__ uint32_t ex2_x2(uint32_t x)
{
    uint32_t d;
    if (BF16) asm("ex2.approx.ftz.bf16x2 %0, %1;" : "=r"(d) : "r"(x));
    else asm("ex2.approx.f16x2 %0, %1;" : "=r"(d) : "r"(x));
    return d;
}
template <bool BF16> __device__ __forceinline__ uint32_t mul_x2(uint32_t a, uint32_t b)
{
    uint32_t d;
    if (BF16) asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    else asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

// Two fp32 values in one 64-bit register pair, and the packed fp32 arithmetic of sm_100 on them (one
// instruction for two lanes of an fma / mul).
__device__ __forceinline__ uint64_t pack2(float lo, float hi)
{
    return (static_cast<uint64_t>(__float_as_uint(hi)) << 32) | __float_as_uint(lo);
}
__device__ __forceinline__ float lo_of(uint64_t v) { return __uint_as_float(static_cast<uint32_t>(v)); }
__device__ __forceinline__ float hi_of(uint64_t v) { return __uint_as_float(static_cast<uint32_t>(v >> 32)); }
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c)
{
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b)
{
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b)
{
    uint64_t d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

__device__ __forceinline__ uint32_t pack16(float a, float b, bool bf16)
{
    if (bf16) {
        __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&t);
    }
    __half2 t = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&t);
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeFn get_encode()
{
    static EncodeFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeFn>(p);
    });
    return fn;
}

inline int ilog2(int x) { int l = 0; while ((1 << l) < x) ++l; return l; }
inline int pow2ceil(int x) { return 1 << ilog2(x); }

// Internal geometry always has three axes; lower ranks get leading axes of size 1.
struct Plan {
    TcParams p;
    int box_q[3], box_kv[3];
};

// Pick the row-tile shape (128 rows) whose column box needs the fewest chunks of `chunk` columns.
inline bool make_plan(const Geo& g, Plan& plan, int chunk = kChunk, bool with_stride = false, bool interleave = false)
{
    TcParams& p = plan.p;
    const int pad = 3 - g.rank;
    for (int a = 0; a < 3; ++a) {
        const int s = a - pad;
        p.L[a] = s >= 0 ? g.L[s] : 1;
        p.K[a] = s >= 0 ? g.K[s] : 1;
        p.dil[a] = s >= 0 ? g.dil[s] : 1;
        p.causal[a] = s >= 0 ? g.causal[s] : 0;
        p.st[a] = (with_stride && s >= 0) ? g.st[s] : 1;
        p.O[a] = (p.L[a] + p.st[a] - 1) / p.st[a];
        if (p.dil[a] > 8) return false;                          // tensor-map element strides, qx0 table
        int gcd = p.dil[a], r = p.st[a];
        while (r) { const int t = gcd % r; gcd = r; r = t; }
        p.qstep[a] = p.st[a] / gcd;
        p.grp_step[a] = gcd;
        p.grp_n[a] = p.dil[a] / gcd;
        p.grp_mul[a] = p.grp_n[a] >= 2 ? (unsigned)((0x100000000ull + p.grp_n[a] - 1) / p.grp_n[a]) : 0u;
        for (int rgrp = 0; rgrp < 8; ++rgrp) {
            p.qx0[a][rgrp] = -1;
            if (rgrp >= p.dil[a]) continue;
            for (int x = 0; x < p.qstep[a]; ++x)
                if ((rgrp + p.dil[a] * x) % p.st[a] == 0) { p.qx0[a][rgrp] = x; break; }
        }
    }
    p.otot = (long long)p.O[0] * p.O[1] * p.O[2];
    long long best = -1;
    for (int t2 = 1; t2 <= 128; t2 *= 2)
        for (int t1 = 1; t1 * t2 <= 128; t1 *= 2) {
            const int t0 = 128 / (t1 * t2);
            const int t[3] = {t0, t1, t2};
            bool fits = true;
            for (int a = 0; a < 3; ++a) {
                if (p.L[a] == 1 && t[a] != 1) fits = false;      // unused axis
                if (t[a] * p.dil[a] * p.qstep[a] > 256) fits = false;     // TMA box limit of the query tile
            }
            if (!fits) continue;
            const int E2 = (t2 - 1) * p.qstep[2] + p.K[2];
            int cb2 = pow2ceil(E2);
            if (cb2 > chunk) cb2 = chunk;
            if (cb2 * p.dil[2] > 256) continue;                  // TMA box limit
            const int E1 = (t1 - 1) * p.qstep[1] + p.K[1];
            int cb1 = chunk / cb2;
            if (p.L[1] == 1) cb1 = 1;
            if (cb1 > pow2ceil(E1)) cb1 = pow2ceil(E1);
            if (cb1 * p.dil[1] > 256) continue;
            int cb0 = chunk / (cb2 * cb1);
            if (p.L[0] == 1 && cb0 != 1) continue;               // would leave the chunk short of columns
            if (cb0 * p.dil[0] > 256) continue;
            const int E0 = (t0 - 1) * p.qstep[0] + p.K[0];
            const long long n = (long long)((E0 + cb0 - 1) / cb0) * ((E1 + cb1 - 1) / cb1) * ((E2 + cb2 - 1) / cb2);
            // prefer fewer chunks, then wider innermost tiles
            if (best < 0 || n < best) {
                best = n;
                for (int a = 0; a < 3; ++a) p.tile[a] = t[a];
                p.cb[0] = cb0; p.cb[1] = cb1; p.cb[2] = cb2;
                p.nchunk[0] = (E0 + cb0 - 1) / cb0; p.nchunk[1] = (E1 + cb1 - 1) / cb1; p.nchunk[2] = (E2 + cb2 - 1) / cb2;
            }
        }
    if (best < 0) return false;
    p.cb0_log = ilog2(p.cb[0]); p.cb1_log = ilog2(p.cb[1]); p.cb2_log = ilog2(p.cb[2]);
    p.tile1_log = ilog2(p.tile[1]); p.tile2_log = ilog2(p.tile[2]);
    p.nchunks = (int)best;
    p.ntiles = 1;
    for (int a = 0; a < 3; ++a) {
        const int lp = (p.L[a] + p.dil[a] - 1) / p.dil[a];
        const int nq = (lp + p.qstep[a] - 1) / p.qstep[a];       // most queries a group can hold along this axis
        p.ntile[a] = (nq + p.tile[a] - 1) / p.tile[a];
        p.ntiles *= p.ntile[a];
        p.ntile_mul[a] = p.ntile[a] >= 2 ? (unsigned)((0x100000000ull + p.ntile[a] - 1) / p.ntile[a]) : 0u;
        p.dil_mul[a] = p.dil[a] >= 2 ? (unsigned)((0x100000000ull + p.dil[a] - 1) / p.dil[a]) : 0u;
        plan.box_q[a] = p.tile[a] * p.dil[a] * p.qstep[a];
        plan.box_kv[a] = p.cb[a] * p.dil[a];
        if (plan.box_q[a] > 256) return false;
    }
    {
        long long blocks = p.ntiles;
        int dmax = 1;
        for (int a = 0; a < 3; ++a) { blocks *= p.grp_n[a]; dmax = p.dil[a] > dmax ? p.dil[a] : dmax; dmax = p.ntile[a] > dmax ? p.ntile[a] : dmax; }
        if (blocks * dmax >= (1ll << 32) || (long long)(p.L[0] + p.L[1] + p.L[2] + dmax) * dmax >= (1ll << 32)) return false;
    }
    for (int a = 0; a < 3; ++a) { p.il[a] = 1; p.il_mul[a] = 0u; }
    if (interleave) {
        // the first (slowest) axis that needs several chunks is the one along which the warps of a
        // tile differ; tensor maps take element strides up to 8
        for (int a = 0; a < 3; ++a) {
            if (p.nchunk[a] <= 1) continue;
            const int il = p.nchunk[a];
            if (p.dil[a] * il <= 8 && p.cb[a] * p.dil[a] * il <= 256) {
                p.il[a] = il;
                p.il_mul[a] = (unsigned)((0x100000000ull + il - 1) / il);
                plan.box_kv[a] = p.cb[a] * p.dil[a] * il;
            }
            break;
        }
    }
    p.dreal = g.D;
    p.split_heads = (g.D != 64 && g.D != 128) ? 1 : 0;
    p.group_mul = g.group >= 2 ? (unsigned)((0x100000000ull + g.group - 1) / g.group) : 0u;
    p.rank = g.rank; p.B = g.B; p.Hq = g.Hq; p.Hkv = g.Hkv; p.group = g.group;
    p.n_extra = g.n_extra;
    p.ngroups = 1;
    for (int a = 0; a < 3; ++a) p.ngroups *= p.grp_n[a];
    p.per_head = (unsigned)p.ntiles * (unsigned)p.ngroups;
    if ((long long)p.per_head * g.B * g.Hq >= (1ll << 31)) return false;
    p.work_q = p.per_head * (unsigned)g.B * (unsigned)g.Hq;
    p.work_kv = p.per_head * (unsigned)g.B * (unsigned)g.Hkv;
    p.scale_log2 = (float)(g.scale * 1.4426950408889634);
    p.scale = (float)g.scale;
    p.extents = g.extents;
    p.ltot = g.ltot;
    p.wait_budget = debug_wait_budget();
    p.inject = debug_inject();
    return true;
}

// 5-D map over [B, X0, X1, X2, heads*D] (innermost first in the arrays below).
inline bool encode_map(CUtensorMap* map, const void* base, bool bf16, const TcParams& p, int heads, int dh,
                const long long strides[3], const int box[3], bool query_lattice = false, bool interleaved = false)
{
    EncodeFn enc = get_encode();
    if (!enc) return false;
    const cuuint64_t tok = (cuuint64_t)strides[1] * 2;
    cuuint64_t dims[5] = {(cuuint64_t)heads * dh, (cuuint64_t)p.L[2], (cuuint64_t)p.L[1], (cuuint64_t)p.L[0], (cuuint64_t)p.B};
    cuuint64_t gstr[4] = {tok, tok * p.L[2], tok * p.L[2] * p.L[1], (cuuint64_t)strides[0] * 2};
    cuuint32_t bx[5] = {64, (cuuint32_t)box[2], (cuuint32_t)box[1], (cuuint32_t)box[0], 1};
    cuuint32_t es[5] = {1, (cuuint32_t)p.dil[2], (cuuint32_t)p.dil[1], (cuuint32_t)p.dil[0], 1};
    if (query_lattice)                                           // strided output: only every qstep-th sub-grid position is a query
        for (int a = 0; a < 3; ++a) es[3 - a] *= (cuuint32_t)p.qstep[a];
    if (interleaved)                                             // chunk columns are il sub-grid positions apart
        for (int a = 0; a < 3; ++a) es[3 - a] *= (cuuint32_t)p.il[a];
    if (p.split_heads) {                                         // [D, H, X2, X1, B]; the leading spatial axis has extent 1
        if (p.L[0] != 1) return false;
        dims[0] = (cuuint64_t)dh; dims[1] = (cuuint64_t)heads; dims[2] = (cuuint64_t)p.L[2]; dims[3] = (cuuint64_t)p.L[1];
        gstr[0] = (cuuint64_t)strides[2] * 2; gstr[1] = tok; gstr[2] = tok * p.L[2];
        bx[1] = 1; bx[2] = (cuuint32_t)box[2]; bx[3] = (cuuint32_t)box[1];
        const cuuint32_t e2 = es[1], e1 = es[2];
        es[1] = 1; es[2] = e2; es[3] = e1;
    }
    for (int i = 1; i < 4; ++i)
        if (es[i] > 8) return false;
    if (dims[4] == 0) return false;
    const CUresult r = enc(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 5,
                           const_cast<void*>(base), dims, gstr, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

// Map over the additional tokens [B, Ne, heads, dh]: same 5-D form, one spatial axis of extent Ne.
inline bool encode_extra_map(CUtensorMap* map, const void* base, bool bf16, int B, int n_extra, int heads,
                             int dh, int box_cols, bool split_heads = false)
{
    EncodeFn enc = get_encode();
    if (!enc || n_extra <= 0) return false;
    const cuuint64_t tok = (cuuint64_t)heads * dh * 2;
    cuuint64_t dims[5] = {(cuuint64_t)heads * dh, (cuuint64_t)n_extra, 1, 1, (cuuint64_t)B};
    cuuint64_t gstr[4] = {tok, tok * n_extra, tok * n_extra, tok * n_extra};
    cuuint32_t bx[5] = {64, (cuuint32_t)box_cols, 1, 1, 1};
    cuuint32_t es[5] = {1, 1, 1, 1, 1};
    if (split_heads) {                                           // [D, H, Ne, 1, B]
        dims[0] = (cuuint64_t)dh; dims[1] = (cuuint64_t)heads; dims[2] = (cuuint64_t)n_extra;
        gstr[0] = (cuuint64_t)dh * 2; gstr[1] = tok; gstr[2] = tok * n_extra;
        bx[1] = 1; bx[2] = (cuuint32_t)box_cols;
    }
    return enc(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 5,
               const_cast<void*>(base), dims, gstr, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Bits [0, n) of a 32-bit word (n may be <= 0 or >= 32).
__device__ __forceinline__ uint32_t low_bits(int n)
{
    return n <= 0 ? 0u : (n >= 32 ? 0xffffffffu : ((1u << n) - 1u));
}

// What piece_word_ranges gives, for chunks that are one run of the innermost axis (cb[0] == cb[1] == 1, not
// interleaved along it): validity bits of columns [32*pc, 32*pc + 32) of chunk (ci[0], ci[1], ci[2]) for a row
// whose window is [f, e) per axis.  A dozen instructions instead of the general form's ranges per axis.
__device__ __forceinline__ bool line_chunks(const TcParams& P) { return P.cb[0] == 1 && P.cb[1] == 1 && P.il[2] == 1; }
__device__ __forceinline__ uint32_t line_word(const TcParams& P, int pc, const int (&ci)[3], const int (&f)[3], const int (&e)[3])
{
    if (ci[0] < f[0] || ci[0] >= e[0] || ci[1] < f[1] || ci[1] >= e[1]) return 0u;
    const int base = ci[2] * P.cb[2] + 32 * pc;
    int lo = f[2] - base, hi = e[2] - base;
    lo = lo > 0 ? lo : 0;
    hi = hi < 32 ? hi : 32;
    return hi > lo ? (low_bits(hi) & ~low_bits(lo)) : 0u;
}

// CTAs of a persistent launch: `per_sm` per multiprocessor, never more than there is work.
inline unsigned persistent_grid(unsigned work, int per_sm)
{
    const unsigned cap = (unsigned)(sm_count() * per_sm);
    return work < cap ? work : cap;
}

// Kernel sizes the tensor-core geometry covers along axis a: every odd size; an even size when the axis
// is not dilated, longer than the kernel and has no per-sample extents (with an even kernel the
// reference's clamped window start depends on the dilation group and can turn negative at L == K).
inline bool kernel_axis_ok(const Geo& g, int a)
{
    return (g.K[a] & 1) || (g.dil[a] == 1 && g.L[a] > g.K[a] && !g.extents);
}

inline bool tc_eligible(int dtype, const Geo& g, const void* q, const void* k, const void* v, bool allow_stride = false)
{
    if (dtype != 1 && dtype != 2) return false;                 // f16 / bf16
    if (g.D < 8 || g.D > 128 || g.D % 8 != 0 || g.Dv != g.D) return false;
    const bool padded = g.D != 64 && g.D != 128;              // zero-padded channels need the head as a map axis of its own
    if (padded && g.rank > 2) return false;
    if (!(g.scale > 0.0)) return false;
    for (int a = 0; a < g.rank; ++a) {
        if (g.st[a] != 1 && !allow_stride) return false;
        if (!kernel_axis_ok(g, a)) return false;
    }
    // heads must be adjacent so that (head, channel) folds into one map dimension
    if (!padded && (g.qs[2] != g.D || g.ks[2] != g.D || g.vs[2] != g.Dv)) return false;
    if (padded && (g.qs[2] % 8 != 0 || g.ks[2] % 8 != 0 || g.vs[2] % 8 != 0)) return false;
    const long long strs[6] = {g.qs[0], g.qs[1], g.ks[0], g.ks[1], g.vs[0], g.vs[1]};
    for (long long s : strs)
        if (s % 8 != 0) return false;                           // 16-byte global strides
    const void* ptrs[3] = {q, k, v};
    for (const void* p : ptrs)
        if (reinterpret_cast<uintptr_t>(p) & 15u) return false;
    return true;
}



} // namespace tcplan
} // namespace natten
