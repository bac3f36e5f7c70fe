// SIMT kernels: the all-feature path (every rank, dtype, head dim, kernel size,
// stride, dilation, per-axis causal, GQA, additional tokens, per-sample extents).
// They serve fp32 / fp64 (where tensor cores would break the 1e-5 parity bound),
// shapes the tcgen05 kernels do not cover, and the split QK / AV ops.
//
// Mapping: one warp per (query, head) for query-centric work and one warp per
// (key, kv head) for the inverse-neighbourhood work.  Inside a warp the score
// phase runs lane-per-neighbour (each lane a full dot product, rows read with
// 16-byte loads) and the accumulate phase runs lane-per-channel (coalesced row
// reads, the weight broadcast by shuffle), so no per-neighbour warp reduction
// is needed.  dK/dV are gathered per key in a fixed order: no float atomics,
// results are bit-reproducible.
#include "simt_kernels.cuh"

#include "device_cache.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math_constants.h>
#include <initializer_list>
#include <type_traits>

namespace natten {

size_t simt_delta_bytes(const Geo& g, size_t acc_size);

namespace {

constexpr int kWarps = 4;
constexpr unsigned kFull = 0xffffffffu;

template <typename T> struct AccOf { using type = float; };
template <> struct AccOf<double> { using type = double; };

__device__ __forceinline__ float to_acc(float x) { return x; }
__device__ __forceinline__ float to_acc(__half x) { return __half2float(x); }
__device__ __forceinline__ float to_acc(__nv_bfloat16 x) { return __bfloat162float(x); }
__device__ __forceinline__ double to_acc(double x) { return x; }

template <typename T, typename A> __device__ __forceinline__ T from_acc(A x);
template <> __device__ __forceinline__ float from_acc<float, float>(float x) { return x; }
template <> __device__ __forceinline__ __half from_acc<__half, float>(float x) { return __float2half_rn(x); }
template <> __device__ __forceinline__ __nv_bfloat16 from_acc<__nv_bfloat16, float>(float x) { return __float2bfloat16_rn(x); }
template <> __device__ __forceinline__ double from_acc<double, double>(double x) { return x; }

__device__ __forceinline__ float exp_acc(float x) { return expf(x); }
__device__ __forceinline__ double exp_acc(double x) { return exp(x); }
__device__ __forceinline__ float log_acc(float x) { return logf(x); }
__device__ __forceinline__ double log_acc(double x) { return log(x); }
template <typename A> __device__ __forceinline__ A neg_inf();
template <> __device__ __forceinline__ float neg_inf<float>() { return -CUDART_INF_F; }
template <> __device__ __forceinline__ double neg_inf<double>() { return -CUDART_INF; }

template <typename A> __device__ __forceinline__ A warp_max(A v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { A t = __shfl_xor_sync(kFull, v, o); v = t > v ? t : v; }
    return v;
}
template <typename A> __device__ __forceinline__ A warp_sum(A v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(kFull, v, o);
    return v;
}
template <typename P> __device__ __forceinline__ const P* shfl_ptr(const P* p, int src)
{
    return reinterpret_cast<const P*>(__shfl_sync(kFull, reinterpret_cast<unsigned long long>(p), src));
}

// dot(staged[0..n), row[0..n)) with 16-byte row loads when the launch allows it.
template <typename T, typename A>
__device__ __forceinline__ A dot_row(const A* __restrict__ staged, const T* __restrict__ row, int n, int vec_ok)
{
    constexpr int V = 16 / sizeof(T);
    A acc = 0;
    if (vec_ok) {
        for (int d = 0; d < n; d += V) {
            const uint4 raw = *reinterpret_cast<const uint4*>(row + d);
            const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
            for (int i = 0; i < V; ++i) acc += staged[d + i] * to_acc(e[i]);
        }
    } else {
        for (int d = 0; d < n; ++d) acc += staged[d] * to_acc(row[d]);
    }
    return acc;
}

struct QueryCtx {
    int b, h, hk;
    long long row;      // (b*otot + o)*Hq + h
    long long pflat;    // flat input position of the query
    int Ls[3], first[3];
    bool inside;
};

// Geometry of the query at output position o (row-major over the output extents) of sample b, head h;
// without kWindows the window starts (c.first) are left out.
template <bool kWindows = true>
__device__ __forceinline__ void decode_at(const Geo& g, int b, long long o, int h, QueryCtx& c)
{
    c.row = ((long long)b * g.otot + o) * g.Hq + h;
    c.h = h;
    c.b = b;
    c.hk = h / g.group;
    c.inside = true;
    int pos[3] = {0, 0, 0};
    // loops over the three axes with the rank as a guard: the small arrays stay in registers
    if (g.otot <= 0x7fffffffll) {                                // 32-bit divisions: the common case
        unsigned o32 = (unsigned)o;
#pragma unroll
        for (int a = 2; a >= 0; --a) {
            if (a >= g.rank) continue;
            const unsigned nx = o32 / (unsigned)g.O[a];
            pos[a] = (int)(o32 - nx * (unsigned)g.O[a]) * g.st[a];
            o32 = nx;
        }
    } else {
#pragma unroll
        for (int a = 2; a >= 0; --a) {
            if (a >= g.rank) continue;
            pos[a] = (int)(o % g.O[a]) * g.st[a];
            o /= g.O[a];
        }
    }
    c.pflat = 0;
#pragma unroll
    for (int a = 0; a < 3; ++a) {
        if (a >= g.rank) continue;
        c.Ls[a] = g.extents ? g.extents[c.b * g.rank + a] : g.L[a];
        if (pos[a] >= c.Ls[a]) c.inside = false;
        c.pflat = c.pflat * g.L[a] + pos[a];
    }
    if constexpr (kWindows) {
#pragma unroll
        for (int a = 0; a < 3; ++a) {
            if (a >= g.rank) continue;
            c.first[a] = c.inside ? axis_first_key(pos[a], c.Ls[a], g.K[a], g.dil[a], g.causal[a]) : 0;
        }
    }
}

__device__ __forceinline__ void decode_query(const Geo& g, long long row, QueryCtx& c)
{
    const int h = (int)(row % g.Hq);
    const long long bo = row / g.Hq;
    decode_at(g, (int)(bo / g.otot), bo % g.otot, h, c);
}

// Flat key position of neighbour slot j (row-major over the per-axis slots).
__device__ __forceinline__ bool slot_key(const Geo& g, const QueryCtx& c, int j, long long& kflat)
{
    int kk[3] = {0, 0, 0};
    for (int a = g.rank - 1; a >= 0; --a) { kk[a] = j % g.K[a]; j /= g.K[a]; }
    bool valid = true;
    kflat = 0;
    for (int a = 0; a < g.rank; ++a) {
        const int pos = c.first[a] + kk[a] * g.dil[a];
        valid = valid && pos >= 0 && pos < c.Ls[a];
        kflat = kflat * g.L[a] + pos;
    }
    return valid;
}

struct KeyCtx {
    int b, hk;
    long long nflat;
    int n[3], Ls[3], base[3], cnt[3];
    int ncand;          // candidate queries (positions) of this key
    bool inside;
};

__device__ __forceinline__ void decode_key(const Geo& g, long long row, KeyCtx& c)
{
    c.hk = (int)(row % g.Hkv);
    long long bn = row / g.Hkv;
    c.nflat = bn % g.ltot;
    c.b = (int)(bn / g.ltot);
    long long n = c.nflat;
    c.inside = true;
    c.ncand = 1;
    for (int a = g.rank - 1; a >= 0; --a) {
        c.n[a] = (int)(n % g.L[a]);
        n /= g.L[a];
        c.Ls[a] = g.extents ? g.extents[c.b * g.rank + a] : g.L[a];
        if (c.n[a] >= c.Ls[a]) c.inside = false;
    }
    for (int a = 0; a < 3; ++a) { c.base[a] = 0; c.cnt[a] = 1; }
    if (c.inside)
        for (int a = 0; a < g.rank; ++a) {
            axis_candidates(c.n[a], c.Ls[a], g.K[a], g.dil[a], g.causal[a], c.base[a], c.cnt[a]);
            c.ncand *= c.cnt[a];
        }
}

// Candidate t (position index inside the candidate box) -> does that query attend
// to this key?  Returns the query's flat output index, flat input position and slot.
__device__ __forceinline__ bool candidate(const Geo& g, const KeyCtx& c, int t,
                                          long long& oflat, long long& pflat, int& slot)
{
    int tt[3] = {0, 0, 0};
    for (int a = g.rank - 1; a >= 0; --a) { tt[a] = t % c.cnt[a]; t /= c.cnt[a]; }
    bool valid = true;
    oflat = 0; pflat = 0; slot = 0;
    for (int a = 0; a < g.rank; ++a) {
        const int p = c.base[a] + tt[a] * g.dil[a];
        if (p % g.st[a] != 0) valid = false;
        const int s = axis_slot(p, c.n[a], c.Ls[a], g.K[a], g.dil[a], g.causal[a]);
        if (s < 0) valid = false;
        oflat = oflat * g.O[a] + p / g.st[a];
        pflat = pflat * g.L[a] + p;
        slot = slot * g.K[a] + s;
    }
    return valid;
}

// ---------------------------------------------------------------------------
// Fused forward
// ---------------------------------------------------------------------------
template <typename T, int NDV>
__global__ void __launch_bounds__(kWarps * 32)
fused_fwd_kernel(const __grid_constant__ Geo g, const T* __restrict__ q, const T* __restrict__ k,
                 const T* __restrict__ v, const T* __restrict__ ek, const T* __restrict__ ev,
                 T* __restrict__ out, typename AccOf<T>::type* __restrict__ lse, long long rows)
{
    using A = typename AccOf<T>::type;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    A* qsh = reinterpret_cast<A*>(smem_raw) + (size_t)warp * g.D;
    const long long row = (long long)blockIdx.x * kWarps + warp;
    if (row >= rows) return;
    QueryCtx c;
    decode_query(g, row, c);
    T* orow = out + row * g.Dv;
    if (!c.inside) {
        for (int d = lane; d < g.Dv; d += 32) orow[d] = from_acc<T, A>(A(0));
        if (lane == 0) lse[row] = A(0);
        return;
    }
    const T* qrow = q + c.b * g.qs[0] + c.pflat * g.qs[1] + c.h * g.qs[2];
    for (int d = lane; d < g.D; d += 32) qsh[d] = to_acc(qrow[d]);
    __syncwarp();

    A m = neg_inf<A>(), l = 0;
    A acc[NDV];
#pragma unroll
    for (int i = 0; i < NDV; ++i) acc[i] = 0;
    const int ntot = g.ktot + g.n_extra;
    const A scale = (A)g.scale;
    for (int base = 0; base < ntot; base += 32) {
        const int j = base + lane;
        const T* krow = nullptr;
        const T* vrow = nullptr;
        bool valid = false;
        if (j < g.ktot) {
            long long kf;
            valid = slot_key(g, c, j, kf);
            if (valid) {
                krow = k + c.b * g.ks[0] + kf * g.ks[1] + c.hk * g.ks[2];
                vrow = v + c.b * g.vs[0] + kf * g.vs[1] + c.hk * g.vs[2];
            }
        } else if (j < ntot) {
            const long long e = ((long long)c.b * g.n_extra + (j - g.ktot)) * g.Hkv + c.hk;
            krow = ek + e * g.D;
            vrow = ev + e * g.Dv;
            valid = true;
        }
        A s = neg_inf<A>();
        if (valid) s = dot_row<T, A>(qsh, krow, g.D, g.vec_ok) * scale;
        const A mx = warp_max(s);
        const A m_new = mx > m ? mx : m;
        if (m_new == neg_inf<A>()) continue;          // nothing valid yet
        const A alpha = (m == neg_inf<A>()) ? A(0) : exp_acc(m - m_new);
        const A p = valid ? exp_acc(s - m_new) : A(0);
        l = l * alpha + warp_sum(p);
#pragma unroll
        for (int i = 0; i < NDV; ++i) acc[i] *= alpha;
        m = m_new;
        unsigned mask = __ballot_sync(kFull, valid);
        while (mask) {
            const int src = __ffs(mask) - 1;
            mask &= mask - 1;
            const A pj = __shfl_sync(kFull, p, src);
            const T* vr = shfl_ptr(vrow, src);
#pragma unroll
            for (int i = 0; i < NDV; ++i) {
                const int d = lane + 32 * i;
                if (d < g.Dv) acc[i] += pj * to_acc(vr[d]);
            }
        }
    }
    const A inv = A(1) / l;
#pragma unroll
    for (int i = 0; i < NDV; ++i) {
        const int d = lane + 32 * i;
        if (d < g.Dv) orow[d] = from_acc<T, A>(acc[i] * inv);
    }
    if (lane == 0) lse[row] = m + log_acc(l);
}

// delta[row] = sum_d out[row,d] * dout[row,d]
template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
delta_kernel(const T* __restrict__ out, const T* __restrict__ dout,
             typename AccOf<T>::type* __restrict__ delta, long long rows, int Dv)
{
    using A = typename AccOf<T>::type;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * kWarps + warp;
    if (row >= rows) return;
    A acc = 0;
    for (int d = lane; d < Dv; d += 32) acc += to_acc(out[row * Dv + d]) * to_acc(dout[row * Dv + d]);
    acc = warp_sum(acc);
    if (lane == 0) delta[row] = acc;
}

// ---------------------------------------------------------------------------
// Fused backward, query side: dQ
// ---------------------------------------------------------------------------
template <typename T, int ND>
__global__ void __launch_bounds__(kWarps * 32)
fused_bwd_dq_kernel(const __grid_constant__ Geo g, const T* __restrict__ q, const T* __restrict__ k,
                    const T* __restrict__ v, const T* __restrict__ ek, const T* __restrict__ ev,
                    const typename AccOf<T>::type* __restrict__ lse,
                    const typename AccOf<T>::type* __restrict__ delta,
                    const T* __restrict__ dout, const typename AccOf<T>::type* __restrict__ dlse,
                    T* __restrict__ dq, long long rows)
{
    using A = typename AccOf<T>::type;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    A* qsh = reinterpret_cast<A*>(smem_raw) + (size_t)warp * (g.D + g.Dv);
    A* dosh = qsh + g.D;
    const long long row = (long long)blockIdx.x * kWarps + warp;
    if (row >= rows) return;
    QueryCtx c;
    decode_query(g, row, c);
    if (!c.inside) return;                       // dq was zero-filled by the launcher
    const T* qrow = q + c.b * g.qs[0] + c.pflat * g.qs[1] + c.h * g.qs[2];
    for (int d = lane; d < g.D; d += 32) qsh[d] = to_acc(qrow[d]);
    for (int d = lane; d < g.Dv; d += 32) dosh[d] = to_acc(dout[row * g.Dv + d]);
    __syncwarp();
    const A lse_i = lse[row];
    const A extra = (dlse ? dlse[row] : A(0)) - delta[row];
    const A scale = (A)g.scale;
    A acc[ND];
#pragma unroll
    for (int i = 0; i < ND; ++i) acc[i] = 0;
    const int ntot = g.ktot + g.n_extra;
    for (int base = 0; base < ntot; base += 32) {
        const int j = base + lane;
        const T* krow = nullptr;
        const T* vrow = nullptr;
        bool valid = false;
        if (j < g.ktot) {
            long long kf;
            valid = slot_key(g, c, j, kf);
            if (valid) {
                krow = k + c.b * g.ks[0] + kf * g.ks[1] + c.hk * g.ks[2];
                vrow = v + c.b * g.vs[0] + kf * g.vs[1] + c.hk * g.vs[2];
            }
        } else if (j < ntot) {
            const long long e = ((long long)c.b * g.n_extra + (j - g.ktot)) * g.Hkv + c.hk;
            krow = ek + e * g.D;
            vrow = ev + e * g.Dv;
            valid = true;
        }
        A ds = 0;
        if (valid) {
            const A s = dot_row<T, A>(qsh, krow, g.D, g.vec_ok) * scale;
            const A p = exp_acc(s - lse_i);
            const A dp = dot_row<T, A>(dosh, vrow, g.Dv, g.vec_ok);
            ds = p * (dp + extra) * scale;
        }
        unsigned mask = __ballot_sync(kFull, valid);
        while (mask) {
            const int src = __ffs(mask) - 1;
            mask &= mask - 1;
            const A dsj = __shfl_sync(kFull, ds, src);
            const T* kr = shfl_ptr(krow, src);
#pragma unroll
            for (int i = 0; i < ND; ++i) {
                const int d = lane + 32 * i;
                if (d < g.D) acc[i] += dsj * to_acc(kr[d]);
            }
        }
    }
    T* dqrow = dq + ((long long)c.b * g.ltot + c.pflat) * g.Hq * g.D + (long long)c.h * g.D;
#pragma unroll
    for (int i = 0; i < ND; ++i) {
        const int d = lane + 32 * i;
        if (d < g.D) dqrow[d] = from_acc<T, A>(acc[i]);
    }
}

// ---------------------------------------------------------------------------
// Fused backward, key side: dK and dV gathered over the inverse neighbourhood
// ---------------------------------------------------------------------------
template <typename T, int ND, int NDV>
__global__ void __launch_bounds__(kWarps * 32)
fused_bwd_dkdv_kernel(const __grid_constant__ Geo g, const T* __restrict__ q, const T* __restrict__ k,
                      const T* __restrict__ v, const typename AccOf<T>::type* __restrict__ lse,
                      const typename AccOf<T>::type* __restrict__ delta, const T* __restrict__ dout,
                      const typename AccOf<T>::type* __restrict__ dlse,
                      T* __restrict__ dk, T* __restrict__ dv, long long rows)
{
    using A = typename AccOf<T>::type;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    A* ksh = reinterpret_cast<A*>(smem_raw) + (size_t)warp * (g.D + g.Dv);
    A* vsh = ksh + g.D;
    const long long row = (long long)blockIdx.x * kWarps + warp;   // (b*ltot + n)*Hkv + hk
    if (row >= rows) return;
    KeyCtx c;
    decode_key(g, row, c);
    T* dkrow = dk + row * g.D;
    T* dvrow = dv + row * g.Dv;
    if (!c.inside) {
        for (int d = lane; d < g.D; d += 32) dkrow[d] = from_acc<T, A>(A(0));
        for (int d = lane; d < g.Dv; d += 32) dvrow[d] = from_acc<T, A>(A(0));
        return;
    }
    const T* krow = k + c.b * g.ks[0] + c.nflat * g.ks[1] + c.hk * g.ks[2];
    const T* vrow = v + c.b * g.vs[0] + c.nflat * g.vs[1] + c.hk * g.vs[2];
    for (int d = lane; d < g.D; d += 32) ksh[d] = to_acc(krow[d]);
    for (int d = lane; d < g.Dv; d += 32) vsh[d] = to_acc(vrow[d]);
    __syncwarp();
    const A scale = (A)g.scale;
    A acck[ND], accv[NDV];
#pragma unroll
    for (int i = 0; i < ND; ++i) acck[i] = 0;
#pragma unroll
    for (int i = 0; i < NDV; ++i) accv[i] = 0;
    const int total = c.ncand * g.group;
    for (int base = 0; base < total; base += 32) {
        const int cnd = base + lane;
        bool valid = false;
        const T* qrow = nullptr;
        const T* dorow = nullptr;
        A p = 0, ds = 0;
        if (cnd < total) {
            const int gi = cnd / c.ncand, t = cnd % c.ncand;
            long long oflat, pflat; int slot;
            valid = candidate(g, c, t, oflat, pflat, slot);
            if (valid) {
                const int h = c.hk * g.group + gi;
                const long long r = ((long long)c.b * g.otot + oflat) * g.Hq + h;
                qrow = q + c.b * g.qs[0] + pflat * g.qs[1] + h * g.qs[2];
                dorow = dout + r * g.Dv;
                const A s = dot_row<T, A>(ksh, qrow, g.D, g.vec_ok) * scale;
                p = exp_acc(s - lse[r]);
                const A dp = dot_row<T, A>(vsh, dorow, g.Dv, g.vec_ok);
                ds = p * (dp - delta[r] + (dlse ? dlse[r] : A(0))) * scale;
            }
        }
        unsigned mask = __ballot_sync(kFull, valid);
        while (mask) {
            const int src = __ffs(mask) - 1;
            mask &= mask - 1;
            const A dsj = __shfl_sync(kFull, ds, src);
            const A pj = __shfl_sync(kFull, p, src);
            const T* qr = shfl_ptr(qrow, src);
            const T* dor = shfl_ptr(dorow, src);
#pragma unroll
            for (int i = 0; i < ND; ++i) {
                const int d = lane + 32 * i;
                if (d < g.D) acck[i] += dsj * to_acc(qr[d]);
            }
#pragma unroll
            for (int i = 0; i < NDV; ++i) {
                const int d = lane + 32 * i;
                if (d < g.Dv) accv[i] += pj * to_acc(dor[d]);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < ND; ++i) {
        const int d = lane + 32 * i;
        if (d < g.D) dkrow[d] = from_acc<T, A>(acck[i]);
    }
#pragma unroll
    for (int i = 0; i < NDV; ++i) {
        const int d = lane + 32 * i;
        if (d < g.Dv) dvrow[d] = from_acc<T, A>(accv[i]);
    }
}

// Gradients of the additional tokens: every query of the sample (and every
// query head of the group) attends to them.  One block per (b, e, hk); warps
// stride over the queries and are reduced in a fixed order through shared memory.
template <typename T, int ND, int NDV>
__global__ void __launch_bounds__(kWarps * 32)
fused_bwd_extra_kernel(const __grid_constant__ Geo g, const T* __restrict__ q,
                       const T* __restrict__ ek, const T* __restrict__ ev,
                       const typename AccOf<T>::type* __restrict__ lse,
                       const typename AccOf<T>::type* __restrict__ delta, const T* __restrict__ dout,
                       const typename AccOf<T>::type* __restrict__ dlse,
                       T* __restrict__ dek, T* __restrict__ dev)
{
    using A = typename AccOf<T>::type;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    A* ksh = reinterpret_cast<A*>(smem_raw);               // D + Dv staged once per block
    A* vsh = ksh + g.D;
    A* red = vsh + g.Dv;                                   // kWarps * (D + Dv)
    const long long row = blockIdx.x;                      // (b*Ne + e)*Hkv + hk
    const int hk = (int)(row % g.Hkv);
    const int b = (int)(row / ((long long)g.Hkv * g.n_extra));
    for (int d = threadIdx.x; d < g.D; d += blockDim.x) ksh[d] = to_acc(ek[row * g.D + d]);
    for (int d = threadIdx.x; d < g.Dv; d += blockDim.x) vsh[d] = to_acc(ev[row * g.Dv + d]);
    __syncthreads();
    const A scale = (A)g.scale;
    A acck[ND], accv[NDV];
#pragma unroll
    for (int i = 0; i < ND; ++i) acck[i] = 0;
#pragma unroll
    for (int i = 0; i < NDV; ++i) accv[i] = 0;
    const long long total = g.otot * g.group;
    for (long long base = (long long)warp * 32; base < total; base += kWarps * 32) {
        const long long cnd = base + lane;
        bool valid = false;
        const T* qrow = nullptr;
        const T* dorow = nullptr;
        A p = 0, ds = 0;
        if (cnd < total) {
            const int gi = (int)(cnd / g.otot);
            const int h = hk * g.group + gi;
            QueryCtx c;
            decode_query(g, ((long long)b * g.otot + cnd % g.otot) * g.Hq + h, c);
            valid = c.inside;
            if (valid) {
                qrow = q + c.b * g.qs[0] + c.pflat * g.qs[1] + c.h * g.qs[2];
                dorow = dout + c.row * g.Dv;
                const A s = dot_row<T, A>(ksh, qrow, g.D, g.vec_ok) * scale;
                p = exp_acc(s - lse[c.row]);
                const A dp = dot_row<T, A>(vsh, dorow, g.Dv, g.vec_ok);
                ds = p * (dp - delta[c.row] + (dlse ? dlse[c.row] : A(0))) * scale;
            }
        }
        unsigned mask = __ballot_sync(kFull, valid);
        while (mask) {
            const int src = __ffs(mask) - 1;
            mask &= mask - 1;
            const A dsj = __shfl_sync(kFull, ds, src);
            const A pj = __shfl_sync(kFull, p, src);
            const T* qr = shfl_ptr(qrow, src);
            const T* dor = shfl_ptr(dorow, src);
#pragma unroll
            for (int i = 0; i < ND; ++i) {
                const int d = lane + 32 * i;
                if (d < g.D) acck[i] += dsj * to_acc(qr[d]);
            }
#pragma unroll
            for (int i = 0; i < NDV; ++i) {
                const int d = lane + 32 * i;
                if (d < g.Dv) accv[i] += pj * to_acc(dor[d]);
            }
        }
    }
    A* mine = red + (size_t)warp * (g.D + g.Dv);
#pragma unroll
    for (int i = 0; i < ND; ++i) { const int d = lane + 32 * i; if (d < g.D) mine[d] = acck[i]; }
#pragma unroll
    for (int i = 0; i < NDV; ++i) { const int d = lane + 32 * i; if (d < g.Dv) mine[g.D + d] = accv[i]; }
    __syncthreads();
    for (int d = threadIdx.x; d < g.D + g.Dv; d += blockDim.x) {
        A s = 0;
        for (int w = 0; w < kWarps; ++w) s += red[(size_t)w * (g.D + g.Dv) + d];
        if (d < g.D) dek[row * g.D + d] = from_acc<T, A>(s);
        else dev[row * g.Dv + (d - g.D)] = from_acc<T, A>(s);
    }
}

// Gradients of the additional tokens, fast path (float accumulation, head dims <= 128).
// A block owns a contiguous segment of (query, head-of-group) pairs of one (batch, kv head) and
// up to kExtraGroup tokens; every query row is read once and kept in registers while the
// tokens' rows sit in shared memory.  Blocks write partial sums that a second kernel adds in
// a fixed order (deterministic, no atomics).
constexpr int kExtraGroup = 16;
constexpr int kExtraSegRows = 1024;

template <typename T, int ND>
__global__ void __launch_bounds__(kWarps * 32)
extra_grad_partial_kernel(const __grid_constant__ Geo g, const T* __restrict__ q, const T* __restrict__ ek,
                          const T* __restrict__ ev, const float* __restrict__ lse,
                          const float* __restrict__ delta, const T* __restrict__ dout,
                          const float* __restrict__ dlse, float* __restrict__ partial, int e0, int ne)
{
    extern __shared__ __align__(128) unsigned char smem_raw[];
    float* eks = reinterpret_cast<float*>(smem_raw);           // [ne][D]
    float* evs = eks + kExtraGroup * g.D;                      // [ne][Dv]
    float* red = evs + kExtraGroup * g.Dv;                     // [ne][D + Dv]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int seg = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
    const int W = g.D + g.Dv;
    for (int i = threadIdx.x; i < ne * g.D; i += blockDim.x)
        eks[i] = to_acc(ek[(((long long)b * g.n_extra + e0 + i / g.D) * g.Hkv + hk) * g.D + i % g.D]);
    for (int i = threadIdx.x; i < ne * g.Dv; i += blockDim.x)
        evs[i] = to_acc(ev[(((long long)b * g.n_extra + e0 + i / g.Dv) * g.Hkv + hk) * g.Dv + i % g.Dv]);
    for (int i = threadIdx.x; i < kExtraGroup * W; i += blockDim.x) red[i] = 0.f;
    __syncthreads();

    float acck[kExtraGroup][ND], accv[kExtraGroup][ND];
#pragma unroll
    for (int e = 0; e < kExtraGroup; ++e)
#pragma unroll
        for (int i = 0; i < ND; ++i) { acck[e][i] = 0.f; accv[e][i] = 0.f; }
    const float scale = (float)g.scale;
    const long long total = g.otot * g.group;
    long long end = (long long)(seg + 1) * kExtraSegRows;
    if (end > total) end = total;
    for (long long cnd = (long long)seg * kExtraSegRows + warp; cnd < end; cnd += kWarps) {
        const int gi = (int)(cnd / g.otot);
        const int h = hk * g.group + gi;
        QueryCtx c;
        decode_query(g, ((long long)b * g.otot + cnd % g.otot) * g.Hq + h, c);
        if (!c.inside) continue;                               // warp-uniform
        const T* qrow = q + c.b * g.qs[0] + c.pflat * g.qs[1] + c.h * g.qs[2];
        const T* dorow = dout + c.row * g.Dv;
        float qr[ND], dor[ND];
#pragma unroll
        for (int i = 0; i < ND; ++i) {
            const int d = lane + 32 * i;
            qr[i] = d < g.D ? to_acc(qrow[d]) : 0.f;
            dor[i] = d < g.Dv ? to_acc(dorow[d]) : 0.f;
        }
        const float lse_i = lse[c.row];
        const float dl = delta[c.row] - (dlse ? dlse[c.row] : 0.f);
#pragma unroll
        for (int e = 0; e < kExtraGroup; ++e) {
            if (e < ne) {
                float sd = 0.f, dp = 0.f;
#pragma unroll
                for (int i = 0; i < ND; ++i) {
                    const int d = lane + 32 * i;
                    if (d < g.D) sd += qr[i] * eks[e * g.D + d];
                    if (d < g.Dv) dp += dor[i] * evs[e * g.Dv + d];
                }
                sd = warp_sum(sd);
                dp = warp_sum(dp);
                const float p = expf(sd * scale - lse_i);
                const float ds = p * (dp - dl) * scale;
#pragma unroll
                for (int i = 0; i < ND; ++i) { acck[e][i] += ds * qr[i]; accv[e][i] += p * dor[i]; }
            }
        }
    }
    // warps add into the shared buffer one after the other (fixed order)
    for (int w = 0; w < kWarps; ++w) {
        if (warp == w) {
#pragma unroll
            for (int e = 0; e < kExtraGroup; ++e) {
                if (e < ne) {
#pragma unroll
                    for (int i = 0; i < ND; ++i) {
                        const int d = lane + 32 * i;
                        if (d < g.D) red[e * W + d] += acck[e][i];
                        if (d < g.Dv) red[e * W + g.D + d] += accv[e][i];
                    }
                }
            }
        }
        __syncthreads();
    }
    float* dst = partial + ((((long long)b * g.Hkv + hk) * gridDim.x + seg) * kExtraGroup) * W;
    for (int i = threadIdx.x; i < ne * W; i += blockDim.x) dst[i] = red[i];
}

// The same partial sums for 16-bit inputs, organised as two small matrix products per tile of
// 64 (query, head-of-group) rows staged in shared memory:
//   phase 1  thread = (row, 4 tokens):   s = q . ek,  dp = dout . ev  ->  p, ds   (shared memory)
//   phase 2  thread = (channel, dEK|dEV): acc[token] += ds[row][token] * q[row][channel]   (or p * dout)
// 256 threads, about 50 registers, 61 KB of shared memory: several blocks per SM, where the
// row-per-warp kernel above keeps 128 accumulators per thread and runs one.
constexpr int kExtraTileRows = 64;

// Stage one tile of query rows and of their output-gradient rows in shared memory, 16 bytes at a time (rows
// outside their sample are zero; head dims up to 128, 256 threads).  All of a thread's loads are issued
// before its first store: with stores to shared memory in between, the loads go out one latency apart.
template <typename T>
__device__ __forceinline__ void stage_extra_rows(const T* __restrict__ q, const T* __restrict__ dout, const long long* qoff,
                                                 const long long* orow, T* qt, T* gt, int D, int Dv, int qstr, int vstr, int tid)
{
    constexpr int kPer = kExtraTileRows * (128 / 8) / 256;      // 16-byte pieces per thread and tensor at head dim 128
    const int nq8 = D / 8, nv8 = Dv / 8;
    // piece index / pieces per row by a multiplication: exact for indices below 4096 and divisors up to 16
    const unsigned mq = (65536u + nq8 - 1) / nq8, mv = (65536u + nv8 - 1) / nv8;
    uint4 vq[kPer], vg[kPer];
    int sq[kPer], sg[kPer];                                     // shared-memory element offsets, -1 = nothing to store
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
        const int i = tid + 256 * j;
        vq[j] = make_uint4(0, 0, 0, 0);
        vg[j] = make_uint4(0, 0, 0, 0);
        sq[j] = -1;
        sg[j] = -1;
        if (i < kExtraTileRows * nq8) {
            const int r = (int)(((unsigned)i * mq) >> 16), c8 = i - r * nq8;
            const long long o = qoff[r];
            sq[j] = r * qstr + 8 * c8;
            if (o >= 0) vq[j] = __ldg(reinterpret_cast<const uint4*>(q + o + 8 * c8));
        }
        if (i < kExtraTileRows * nv8) {
            const int r = (int)(((unsigned)i * mv) >> 16), c8 = i - r * nv8;
            sg[j] = r * vstr + 8 * c8;
            if (qoff[r] >= 0) vg[j] = __ldg(reinterpret_cast<const uint4*>(dout + orow[r] * Dv + 8 * c8));
        }
    }
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
        if (sq[j] >= 0) *reinterpret_cast<uint4*>(qt + sq[j]) = vq[j];
        if (sg[j] >= 0) *reinterpret_cast<uint4*>(gt + sg[j]) = vg[j];
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
extra_grad_tile_kernel(const __grid_constant__ Geo g, const T* __restrict__ q, const T* __restrict__ ek,
                       const T* __restrict__ ev, const float* __restrict__ lse,
                       const float* __restrict__ delta, const T* __restrict__ dout,
                       const float* __restrict__ dlse, float* __restrict__ partial, int e0, int ne)
{
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int D = g.D, Dv = g.Dv, W = D + Dv;
    const int qstr = D + 8, vstr = Dv + 8;                     // padded row strides (elements): no bank conflicts
    T* qt = reinterpret_cast<T*>(smem_raw);                     // [64][qstr]
    T* gt = qt + kExtraTileRows * qstr;                         // [64][vstr]
    float* eks = reinterpret_cast<float*>(gt + kExtraTileRows * vstr);   // [16][D]
    float* evs = eks + kExtraGroup * D;                         // [16][Dv]
    float* pp = evs + kExtraGroup * Dv;                         // [64][16]  p
    float* dss = pp + kExtraTileRows * kExtraGroup;             // [64][16]  ds
    float* rl = dss + kExtraTileRows * kExtraGroup;             // [64] lse
    float* rd = rl + kExtraTileRows;                            // [64] delta
    long long* qoff = reinterpret_cast<long long*>(rd + kExtraTileRows);   // [64] element offset of the q row, -1 = no row
    long long* orow = qoff + kExtraTileRows;                    // [64] row of dout / lse / delta

    const int tid = threadIdx.x;
    const int seg = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
    for (int i = tid; i < kExtraGroup * D; i += 256)
        eks[i] = (i / D < ne) ? to_acc(ek[(((long long)b * g.n_extra + e0 + i / D) * g.Hkv + hk) * D + i % D]) : 0.f;
    for (int i = tid; i < kExtraGroup * Dv; i += 256)
        evs[i] = (i / Dv < ne) ? to_acc(ev[(((long long)b * g.n_extra + e0 + i / Dv) * g.Hkv + hk) * Dv + i % Dv]) : 0.f;

    float acc[kExtraGroup];
#pragma unroll
    for (int e = 0; e < kExtraGroup; ++e) acc[e] = 0.f;
    const float scale = (float)g.scale;
    const long long total = g.otot * g.group;
    long long end = (long long)(seg + 1) * kExtraSegRows;
    if (end > total) end = total;

    for (long long base = (long long)seg * kExtraSegRows; base < end; base += kExtraTileRows) {
        __syncthreads();                                        // the previous tile has been consumed
        // ---- which rows, where ----
        bool mine_inside = false;
        if (tid < kExtraTileRows) {
            const long long cnd = base + tid;
            long long qo = -1, ro = 0;
            if (cnd < end) {
                int gi;
                long long o;
                if (total <= 0x7fffffffll) { gi = (int)((unsigned)cnd / (unsigned)g.otot); o = (long long)((unsigned)cnd - (unsigned)gi * (unsigned)g.otot); }
                else { gi = (int)(cnd / g.otot); o = cnd % g.otot; }
                QueryCtx c;
                decode_at<false>(g, b, o, hk * g.group + gi, c);
                if (c.inside) {
                    qo = c.b * g.qs[0] + c.pflat * g.qs[1] + c.h * g.qs[2];
                    ro = c.row;
                    mine_inside = true;
                }
            }
            qoff[tid] = qo;
            orow[tid] = ro;
            rl[tid] = mine_inside ? lse[ro] : 0.f;
            rd[tid] = mine_inside ? delta[ro] - (dlse ? dlse[ro] : 0.f) : 0.f;
        }
        if (!__syncthreads_or(mine_inside ? 1 : 0)) continue;   // nothing of this tile is inside its sample
        stage_extra_rows(q, dout, qoff, orow, qt, gt, D, Dv, qstr, vstr, tid);
        __syncthreads();
        // ---- phase 1: probabilities and dS of 4 tokens for one row ----
        {
            const int r = tid & (kExtraTileRows - 1), eg = tid >> 6;
            float sv[4] = {0.f, 0.f, 0.f, 0.f}, dp[4] = {0.f, 0.f, 0.f, 0.f};
            for (int c8 = 0; c8 < D / 8; ++c8) {
                const uint4 raw = *reinterpret_cast<const uint4*>(qt + r * qstr + 8 * c8);
                const T* x = reinterpret_cast<const T*>(&raw);
                float xf[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) xf[i] = to_acc(x[i]);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float4 a = *reinterpret_cast<const float4*>(eks + (4 * eg + j) * D + 8 * c8);
                    const float4 c = *reinterpret_cast<const float4*>(eks + (4 * eg + j) * D + 8 * c8 + 4);
                    sv[j] += xf[0] * a.x + xf[1] * a.y + xf[2] * a.z + xf[3] * a.w + xf[4] * c.x + xf[5] * c.y + xf[6] * c.z + xf[7] * c.w;
                }
            }
            for (int c8 = 0; c8 < Dv / 8; ++c8) {
                const uint4 raw = *reinterpret_cast<const uint4*>(gt + r * vstr + 8 * c8);
                const T* x = reinterpret_cast<const T*>(&raw);
                float xf[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) xf[i] = to_acc(x[i]);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float4 a = *reinterpret_cast<const float4*>(evs + (4 * eg + j) * Dv + 8 * c8);
                    const float4 c = *reinterpret_cast<const float4*>(evs + (4 * eg + j) * Dv + 8 * c8 + 4);
                    dp[j] += xf[0] * a.x + xf[1] * a.y + xf[2] * a.z + xf[3] * a.w + xf[4] * c.x + xf[5] * c.y + xf[6] * c.z + xf[7] * c.w;
                }
            }
            const bool live = qoff[r] >= 0;
            float4 pv, dv;
            float* pa = &pv.x;
            float* da = &dv.x;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const bool on = live && 4 * eg + j < ne;
                const float pj = on ? expf(sv[j] * scale - rl[r]) : 0.f;
                pa[j] = pj;
                da[j] = on ? pj * (dp[j] - rd[r]) * scale : 0.f;
            }
            *reinterpret_cast<float4*>(pp + r * kExtraGroup + 4 * eg) = pv;
            *reinterpret_cast<float4*>(dss + r * kExtraGroup + 4 * eg) = dv;
        }
        __syncthreads();
        // ---- phase 2: one channel of dEK (threads 0-127) or dEV (128-255), all 16 tokens ----
        {
            const int which = tid >> 7, d = tid & 127;
            if (d < (which ? Dv : D)) {
                const T* tile = which ? gt : qt;
                const int str = which ? vstr : qstr;
                const float* wsrc = which ? pp : dss;
#pragma unroll 4
                for (int r = 0; r < kExtraTileRows; ++r) {
                    const float x = to_acc(tile[r * str + d]);
                    const float4* w4 = reinterpret_cast<const float4*>(wsrc + r * kExtraGroup);
#pragma unroll
                    for (int k4 = 0; k4 < 4; ++k4) {
                        const float4 w = w4[k4];
                        acc[4 * k4] += w.x * x;
                        acc[4 * k4 + 1] += w.y * x;
                        acc[4 * k4 + 2] += w.z * x;
                        acc[4 * k4 + 3] += w.w * x;
                    }
                }
            }
        }
    }
    // ---- this block's partial sums: [token][D | Dv] ----
    {
        const int which = tid >> 7, d = tid & 127;
        float* dst = partial + ((((long long)b * g.Hkv + hk) * gridDim.x + seg) * kExtraGroup) * W;
        if (d < (which ? Dv : D)) {
#pragma unroll
            for (int e = 0; e < kExtraGroup; ++e)
                if (e < ne) dst[e * W + (which ? D + d : d)] = acc[e];
        }
    }
}

template <typename T>
__global__ void extra_grad_reduce_kernel(const __grid_constant__ Geo g, const float* __restrict__ partial,
                                         int nseg, int e0, int ne, T* __restrict__ dek, T* __restrict__ dev)
{
    const int W = g.D + g.Dv;
    const long long n = (long long)g.B * g.Hkv * ne * W;
    const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= n) return;
    const int d = (int)(t % W);
    const int e = (int)((t / W) % ne);
    const long long bh = t / ((long long)W * ne);              // b * Hkv + hk
    float acc = 0.f;
    for (int sgm = 0; sgm < nseg; ++sgm) acc += partial[((bh * nseg + sgm) * kExtraGroup + e) * W + d];
    const int hk = (int)(bh % g.Hkv);
    const long long b = bh / g.Hkv;
    const long long tok = (b * g.n_extra + e0 + e) * g.Hkv + hk;
    if (d < g.D) dek[tok * g.D + d] = from_acc<T, float>(acc);
    else dev[tok * g.Dv + (d - g.D)] = from_acc<T, float>(acc);
}

// ---------------------------------------------------------------------------
// Split QK
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
qk_fwd_kernel(const __grid_constant__ Geo g, const T* __restrict__ q, const T* __restrict__ k,
              T* __restrict__ logits, long long rows)
{
    using A = typename AccOf<T>::type;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    A* qsh = reinterpret_cast<A*>(smem_raw) + (size_t)warp * g.D;
    const long long row = (long long)blockIdx.x * kWarps + warp;
    if (row >= rows) return;
    QueryCtx c;
    decode_query(g, row, c);
    const T* qrow = q + c.b * g.qs[0] + c.pflat * g.qs[1] + c.h * g.qs[2];
    for (int d = lane; d < g.D; d += 32) qsh[d] = to_acc(qrow[d]);
    __syncwarp();
    for (int j = lane; j < g.ktot; j += 32) {
        long long kf;
        A val = neg_inf<A>();
        if (slot_key(g, c, j, kf))
            val = dot_row<T, A>(qsh, k + c.b * g.ks[0] + kf * g.ks[1] + c.hk * g.ks[2], g.D, g.vec_ok);
        if (g.has_scale) val *= (A)g.scale;
        logits[row * g.ktot + j] = from_acc<T, A>(val);
    }
}

template <typename T, int ND>
__global__ void __launch_bounds__(kWarps * 32)
qk_bwd_dq_kernel(const __grid_constant__ Geo g, const T* __restrict__ k, const T* __restrict__ dlogits,
                 T* __restrict__ dq, long long rows)
{
    using A = typename AccOf<T>::type;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * kWarps + warp;
    if (row >= rows) return;
    QueryCtx c;
    decode_query(g, row, c);
    const A scale = g.has_scale ? (A)g.scale : A(1);
    A acc[ND];
#pragma unroll
    for (int i = 0; i < ND; ++i) acc[i] = 0;
    for (int j = 0; j < g.ktot; ++j) {
        long long kf;
        if (!slot_key(g, c, j, kf)) continue;               // warp-uniform
        const A w = to_acc(dlogits[row * g.ktot + j]) * scale;
        const T* kr = k + c.b * g.ks[0] + kf * g.ks[1] + c.hk * g.ks[2];
#pragma unroll
        for (int i = 0; i < ND; ++i) {
            const int d = lane + 32 * i;
            if (d < g.D) acc[i] += w * to_acc(kr[d]);
        }
    }
    T* dqrow = dq + ((long long)c.b * g.ltot + c.pflat) * g.Hq * g.D + (long long)c.h * g.D;
#pragma unroll
    for (int i = 0; i < ND; ++i) {
        const int d = lane + 32 * i;
        if (d < g.D) dqrow[d] = from_acc<T, A>(acc[i]);
    }
}

// dK (QK backward) and dV (AV backward) share one gather: for every query that
// attends to the key, weight[query, slot] * row[query].
template <typename T, int ND>
__global__ void __launch_bounds__(kWarps * 32)
inverse_gather_kernel(const __grid_constant__ Geo g, const T* __restrict__ weights,
                      const T* __restrict__ rows_src, long long src_bs, long long src_ts, long long src_hs,
                      int src_is_query_input, int width, double wscale, T* __restrict__ dst, long long rows)
{
    using A = typename AccOf<T>::type;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * kWarps + warp;   // (b*ltot + n)*Hkv + hk
    if (row >= rows) return;
    KeyCtx c;
    decode_key(g, row, c);
    A acc[ND];
#pragma unroll
    for (int i = 0; i < ND; ++i) acc[i] = 0;
    const int total = c.inside ? c.ncand * g.group : 0;
    for (int base = 0; base < total; base += 32) {
        const int cnd = base + lane;
        bool valid = false;
        const T* src = nullptr;
        A w = 0;
        if (cnd < total) {
            const int gi = cnd / c.ncand, t = cnd % c.ncand;
            long long oflat, pflat; int slot;
            valid = candidate(g, c, t, oflat, pflat, slot);
            if (valid) {
                const int h = c.hk * g.group + gi;
                const long long r = ((long long)c.b * g.otot + oflat) * g.Hq + h;
                w = to_acc(weights[r * g.ktot + slot]) * (A)wscale;
                // source row: q (indexed by input position, strided) or dout (by output row)
                src = src_is_query_input ? rows_src + c.b * src_bs + pflat * src_ts + h * src_hs
                                         : rows_src + r * (long long)width;
            }
        }
        unsigned mask = __ballot_sync(kFull, valid);
        while (mask) {
            const int s = __ffs(mask) - 1;
            mask &= mask - 1;
            const A wj = __shfl_sync(kFull, w, s);
            const T* sr = shfl_ptr(src, s);
#pragma unroll
            for (int i = 0; i < ND; ++i) {
                const int d = lane + 32 * i;
                if (d < width) acc[i] += wj * to_acc(sr[d]);
            }
        }
    }
    T* drow = dst + row * width;
#pragma unroll
    for (int i = 0; i < ND; ++i) {
        const int d = lane + 32 * i;
        if (d < width) drow[d] = from_acc<T, A>(acc[i]);
    }
}

// ---------------------------------------------------------------------------
// Split AV
// ---------------------------------------------------------------------------
template <typename T, int NDV>
__global__ void __launch_bounds__(kWarps * 32)
av_fwd_kernel(const __grid_constant__ Geo g, const T* __restrict__ attn, const T* __restrict__ v,
              T* __restrict__ out, long long rows)
{
    using A = typename AccOf<T>::type;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * kWarps + warp;
    if (row >= rows) return;
    QueryCtx c;
    decode_query(g, row, c);
    A acc[NDV];
#pragma unroll
    for (int i = 0; i < NDV; ++i) acc[i] = 0;
    for (int j = 0; j < g.ktot; ++j) {
        long long kf;
        if (!slot_key(g, c, j, kf)) continue;
        const A w = to_acc(attn[row * g.ktot + j]);
        const T* vr = v + c.b * g.vs[0] + kf * g.vs[1] + c.hk * g.vs[2];
#pragma unroll
        for (int i = 0; i < NDV; ++i) {
            const int d = lane + 32 * i;
            if (d < g.Dv) acc[i] += w * to_acc(vr[d]);
        }
    }
#pragma unroll
    for (int i = 0; i < NDV; ++i) {
        const int d = lane + 32 * i;
        if (d < g.Dv) out[row * g.Dv + d] = from_acc<T, A>(acc[i]);
    }
}

template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
av_bwd_dattn_kernel(const __grid_constant__ Geo g, const T* __restrict__ v, const T* __restrict__ dout,
                    T* __restrict__ dattn, long long rows)
{
    using A = typename AccOf<T>::type;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    A* dosh = reinterpret_cast<A*>(smem_raw) + (size_t)warp * g.Dv;
    const long long row = (long long)blockIdx.x * kWarps + warp;
    if (row >= rows) return;
    QueryCtx c;
    decode_query(g, row, c);
    for (int d = lane; d < g.Dv; d += 32) dosh[d] = to_acc(dout[row * g.Dv + d]);
    __syncwarp();
    for (int j = lane; j < g.ktot; j += 32) {
        long long kf;
        A val = 0;
        if (slot_key(g, c, j, kf))
            val = dot_row<T, A>(dosh, v + c.b * g.vs[0] + kf * g.vs[1] + c.hk * g.vs[2], g.Dv, g.vec_ok);
        dattn[row * g.ktot + j] = from_acc<T, A>(val);
    }
}

// ---------------------------------------------------------------------------
// Split ops, vectorised variants for 16-bit tensors whose rows can be read 16 bytes at a time
// (head dim 32 / 64 / 128 / 256, strides multiples of 8 elements).  A warp still owns one
// (query, head) or (key, kv head) row, but LPR = D/8 lanes share one source row (16 bytes each),
// so one load instruction covers 32/LPR whole rows instead of 32 scattered 2-byte pieces, and
// the neighbour offsets are worked out once per row (lane per slot) instead of per channel.
// ---------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ void unpack8(const uint4& raw, float (&f)[8])
{
    const T* x = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = to_acc(x[i]);
}

template <typename T>
__device__ __forceinline__ uint4 pack8(const float (&f)[8])
{
    uint4 raw;
    T* x = reinterpret_cast<T*>(&raw);
#pragma unroll
    for (int i = 0; i < 8; ++i) x[i] = from_acc<T, float>(f[i]);
    return raw;
}

// Element offsets (inside one batch) of a query's neighbours, one per slot; -1 = masked.
__device__ __forceinline__ void neighbour_offsets(const Geo& g, const QueryCtx& c, long long token_stride,
                                                  int lane, int* koff)
{
    for (int j = lane; j < g.ktot; j += 32) {
        long long kf;
        koff[j] = slot_key(g, c, j, kf) ? (int)(kf * token_stride) : -1;
    }
    __syncwarp();
}

// out[row, j] = scale * <x[row], y[neighbour j]>     (QK forward; AV backward w.r.t. attn)
template <typename T, int LPR>
__global__ void __launch_bounds__(kWarps * 32)
dot_neighbours_vec_kernel(const __grid_constant__ Geo g, const T* __restrict__ x, long long xbs, long long xts,
                          long long xhs, int x_by_position, int D, const T* __restrict__ y, long long ybs,
                          long long yts, long long yhs, float scale, int masked_is_neg_inf,
                          T* __restrict__ out, long long rows)
{
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int* koff = reinterpret_cast<int*>(smem_raw) + (size_t)warp * g.ktot;
    const long long row = (long long)blockIdx.x * kWarps + warp;
    if (row >= rows) return;
    QueryCtx c;
    decode_query(g, row, c);
    neighbour_offsets(g, c, yts, lane, koff);
    constexpr int G = 32 / LPR;
    const int gl = lane % LPR, gi = lane / LPR;
    const T* xrow = x_by_position ? x + c.b * xbs + c.pflat * xts + c.h * xhs : x + row * (long long)D;
    float xf[8];
    unpack8<T>(*reinterpret_cast<const uint4*>(xrow + 8 * gl), xf);
    const T* ybase = y + c.b * ybs + c.hk * yhs + 8 * gl;
    const float fill = masked_is_neg_inf ? -INFINITY : 0.f;
    for (int j0 = 0; j0 < g.ktot; j0 += G) {
        const int j = j0 + gi;
        const int off = j < g.ktot ? koff[j] : -1;
        float d = 0.f;
        if (off >= 0) {
            float yf[8];
            unpack8<T>(*reinterpret_cast<const uint4*>(ybase + off), yf);
#pragma unroll
            for (int i = 0; i < 8; ++i) d = fmaf(xf[i], yf[i], d);
        }
#pragma unroll
        for (int m = LPR / 2; m > 0; m >>= 1) d += __shfl_xor_sync(kFull, d, m);
        if (gl == 0 && j < g.ktot) out[row * g.ktot + j] = from_acc<T, float>(off >= 0 ? d * scale : fill);
    }
}

// out[row] = scale * sum_j w[row, j] * y[neighbour j]   (AV forward; QK backward w.r.t. q)
template <typename T, int LPR>
__global__ void __launch_bounds__(kWarps * 32)
sum_neighbours_vec_kernel(const __grid_constant__ Geo g, const T* __restrict__ w, const T* __restrict__ y,
                          long long ybs, long long yts, long long yhs, int D, float scale,
                          int out_by_position, T* __restrict__ out, long long rows)
{
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int* koff = reinterpret_cast<int*>(smem_raw) + (size_t)warp * g.ktot;
    const long long row = (long long)blockIdx.x * kWarps + warp;
    if (row >= rows) return;
    QueryCtx c;
    decode_query(g, row, c);
    neighbour_offsets(g, c, yts, lane, koff);
    constexpr int G = 32 / LPR;
    const int gl = lane % LPR, gi = lane / LPR;
    const T* ybase = y + c.b * ybs + c.hk * yhs + 8 * gl;
    const T* wrow = w + row * g.ktot;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    for (int j0 = 0; j0 < g.ktot; j0 += G) {
        const int j = j0 + gi;
        const int off = j < g.ktot ? koff[j] : -1;
        if (off >= 0) {
            const float wj = to_acc(wrow[j]);
            float yf[8];
            unpack8<T>(*reinterpret_cast<const uint4*>(ybase + off), yf);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = fmaf(wj, yf[i], acc[i]);
        }
    }
#pragma unroll
    for (int m = LPR; m < 32; m <<= 1)
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += __shfl_xor_sync(kFull, acc[i], m);
    if (gi == 0) {
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] *= scale;
        T* orow = out_by_position ? out + (((long long)c.b * g.ltot + c.pflat) * g.Hq + c.h) * D : out + row * (long long)D;
        *reinterpret_cast<uint4*>(orow + 8 * gl) = pack8<T>(acc);
    }
}

// dst[key] = wscale * sum over the queries that attend to the key of weight[query, slot] * src[query]
// (dK of the QK backward, dV of the AV backward).
template <typename T, int LPR>
__global__ void __launch_bounds__(kWarps * 32)
inverse_gather_vec_kernel(const __grid_constant__ Geo g, const T* __restrict__ weights,
                          const T* __restrict__ rows_src, long long src_bs, long long src_ts, long long src_hs,
                          int src_is_query_input, int width, float wscale, T* __restrict__ dst, long long rows)
{
    __shared__ long long s_off[kWarps][32];
    __shared__ float s_w[kWarps][32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * kWarps + warp;   // (b*ltot + n)*Hkv + hk
    if (row >= rows) return;
    KeyCtx c;
    decode_key(g, row, c);
    constexpr int G = 32 / LPR;
    const int gl = lane % LPR, gi = lane / LPR;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    const int total = c.inside ? c.ncand * g.group : 0;
    for (int base = 0; base < total; base += 32) {
        const int cnd = base + lane;
        bool valid = false;
        long long off = 0;
        float wv = 0.f;
        if (cnd < total) {
            const int gidx = cnd / c.ncand, t = cnd % c.ncand;
            long long oflat, pflat; int slot;
            valid = candidate(g, c, t, oflat, pflat, slot);
            if (valid) {
                const int h = c.hk * g.group + gidx;
                const long long r = ((long long)c.b * g.otot + oflat) * g.Hq + h;
                wv = to_acc(weights[r * g.ktot + slot]);
                off = src_is_query_input ? c.b * src_bs + pflat * src_ts + h * src_hs : r * (long long)width;
            }
        }
        // compact the valid candidates of this batch of 32 into the warp's list (fixed order)
        const unsigned mask = __ballot_sync(kFull, valid);
        const int n = __popc(mask);
        if (valid) {
            const int pos = __popc(mask & ((1u << lane) - 1u));
            s_off[warp][pos] = off;
            s_w[warp][pos] = wv;
        }
        __syncwarp();
        for (int i0 = 0; i0 < n; i0 += G) {
            const int i = i0 + gi;
            if (i < n) {
                float yf[8];
                unpack8<T>(*reinterpret_cast<const uint4*>(rows_src + s_off[warp][i] + 8 * gl), yf);
                const float wj = s_w[warp][i];
#pragma unroll
                for (int u = 0; u < 8; ++u) acc[u] = fmaf(wj, yf[u], acc[u]);
            }
        }
        __syncwarp();
    }
#pragma unroll
    for (int m = LPR; m < 32; m <<= 1)
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += __shfl_xor_sync(kFull, acc[i], m);
    if (gi == 0) {
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] *= wscale;
        *reinterpret_cast<uint4*>(dst + row * (long long)width + 8 * gl) = pack8<T>(acc);
    }
}

// Can the vectorised split kernels serve this problem?  (16-bit T is checked by the callers.)
inline bool split_vec_ok(const Geo& g, int D, std::initializer_list<const void*> ptrs,
                         std::initializer_list<long long> strides, long long token_stride)
{
    if (D != 32 && D != 64 && D != 128 && D != 256) return false;
    for (const void* p : ptrs)
        if (reinterpret_cast<uintptr_t>(p) & 15u) return false;
    for (long long st : strides)
        if (st % 8 != 0) return false;
    if ((long long)g.ktot * kWarps * (long long)sizeof(int) > 48 * 1024) return false;
    return g.ltot * token_stride < (1ll << 31);                   // neighbour offsets inside a batch are 32-bit
}

#define NATTEN_DISPATCH_LPR(D, LPR, ...)                                  \
    do {                                                                  \
        if ((D) == 32) { constexpr int LPR = 4; __VA_ARGS__; }            \
        else if ((D) == 64) { constexpr int LPR = 8; __VA_ARGS__; }       \
        else if ((D) == 128) { constexpr int LPR = 16; __VA_ARGS__; }     \
        else { constexpr int LPR = 32; __VA_ARGS__; }                     \
    } while (0)

// ---------------------------------------------------------------------------
// Launch helpers
// ---------------------------------------------------------------------------
unsigned long long g_launches = 0;

inline unsigned grid_for(long long rows) { return (unsigned)((rows + kWarps - 1) / kWarps); }

#define NATTEN_DISPATCH_N(n, NAME, ...)                                     \
    do {                                                                    \
        if ((n) <= 32) { constexpr int NAME = 1; __VA_ARGS__; }             \
        else if ((n) <= 64) { constexpr int NAME = 2; __VA_ARGS__; }        \
        else if ((n) <= 128) { constexpr int NAME = 4; __VA_ARGS__; }       \
        else { constexpr int NAME = 8; __VA_ARGS__; }                       \
    } while (0)


// Warp-level tensor-core helpers for the kernel below: 8 x 8 16-bit matrices from shared memory (every row
// address 16-byte aligned) and the m16n8k16 product with fp32 accumulation.
__device__ __forceinline__ uint32_t shared_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x2(uint32_t& r0, uint32_t& r1, uint32_t addr)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}
template <typename T>
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
    if constexpr (std::is_same<T, __half>::value)
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    else
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <typename T> __device__ __forceinline__ uint32_t pack_pair(float lo, float hi)
{
    const T a = from_acc<T, float>(lo), b = from_acc<T, float>(hi);
    return (uint32_t)(*reinterpret_cast<const unsigned short*>(&a)) | ((uint32_t)(*reinterpret_cast<const unsigned short*>(&b)) << 16);
}

// The same partial sums with the four small matrix products of a tile on the warp-level tensor-core path
// (m16n8k16 fragments fed by ldmatrix; the additional tokens are the 16-wide side of every product):
//   phase 1  warp w takes the 16 rows of block w & 3 and the 8 tokens of half w >> 2:  S = Qt Ek^T and
//            dP = Gt Ev^T over the head dim, then, still in registers, p = exp(S*scale - lse) and
//            ds = p (dP - delta) scale, rounded to the tensors' 16-bit type like the probabilities of the
//            fused kernels and written as [row][token] tiles
//   phase 2  dEk += ds^T Qt, dEv += p^T Gt      [16 tokens x head dim], K = 64 rows     (warp w: channels 16w .. 16w+15)
// The accumulators of phase 2 stay in registers across the block's tiles.  Head dims: multiples of 16 up to 128.
template <typename T>
__global__ void __launch_bounds__(256, 3)
extra_grad_mma_kernel(const __grid_constant__ Geo g, const T* __restrict__ q, const T* __restrict__ ek,
                      const T* __restrict__ ev, const float* __restrict__ lse,
                      const float* __restrict__ delta, const T* __restrict__ dout,
                      const float* __restrict__ dlse, float* __restrict__ partial, int e0, int ne)
{
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int D = g.D, Dv = g.Dv, W = D + Dv;
    const int qstr = D + 8, vstr = Dv + 8;                     // padded row strides (elements; 16-byte multiples)
    constexpr int kPStr = kExtraGroup + 8;                      // row stride of the 16-bit p / ds tiles
    T* qt = reinterpret_cast<T*>(smem_raw);                     // [64][qstr]
    T* gt = qt + kExtraTileRows * qstr;                         // [64][vstr]
    T* ekt = gt + kExtraTileRows * vstr;                        // [16][qstr]   (tokens past ne are zero)
    T* evt = ekt + kExtraGroup * qstr;                          // [16][vstr]
    T* pt = evt + kExtraGroup * vstr;                           // [64][kPStr]  p
    T* dst = pt + kExtraTileRows * kPStr;                       // [64][kPStr]  ds
    float* rl = reinterpret_cast<float*>(dst + kExtraTileRows * kPStr);      // [64] lse
    float* rd = rl + kExtraTileRows;                            // [64] delta
    long long* qoff = reinterpret_cast<long long*>(rd + kExtraTileRows);   // [64] element offset of the q row, -1 = no row
    long long* orow = qoff + kExtraTileRows;                    // [64] row of dout / lse / delta

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int seg = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
    // the tokens' rows, 16 bytes at a time
    for (int i = tid; i < kExtraGroup * (D / 8); i += 256) {
        const int e = i / (D / 8), c8 = i - e * (D / 8);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (e < ne) v = __ldg(reinterpret_cast<const uint4*>(ek + (((long long)b * g.n_extra + e0 + e) * g.Hkv + hk) * D + 8 * c8));
        *reinterpret_cast<uint4*>(ekt + e * qstr + 8 * c8) = v;
    }
    for (int i = tid; i < kExtraGroup * (Dv / 8); i += 256) {
        const int e = i / (Dv / 8), c8 = i - e * (Dv / 8);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (e < ne) v = __ldg(reinterpret_cast<const uint4*>(ev + (((long long)b * g.n_extra + e0 + e) * g.Hkv + hk) * Dv + 8 * c8));
        *reinterpret_cast<uint4*>(evt + e * vstr + 8 * c8) = v;
    }

    float acc_k[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}}, acc_v[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    const float scale = (float)g.scale;
    const long long total = g.otot * g.group;
    long long end = (long long)(seg + 1) * kExtraSegRows;
    if (end > total) end = total;
    const int lr = lane & 7, lm = lane >> 3;                   // row inside an 8 x 8 matrix, matrix of the ldmatrix group
    const int fg = lane >> 2, ft = lane & 3;                   // fragment row and column pair of this lane

    for (long long base = (long long)seg * kExtraSegRows; base < end; base += kExtraTileRows) {
        __syncthreads();                                        // the previous tile has been consumed
        bool mine_inside = false;
        long long my_row = 0;
        if (tid < kExtraTileRows) {
            const long long cnd = base + tid;
            long long qo = -1, ro = 0;
            if (cnd < end) {
                int gi;
                long long o;
                // the heads of the group are the fast index: a tile reads group x D contiguous channels per position
                if (total <= 0x7fffffffll) { const unsigned o32 = (unsigned)cnd / (unsigned)g.group; gi = (int)((unsigned)cnd - o32 * (unsigned)g.group); o = (long long)o32; }
                else { o = cnd / g.group; gi = (int)(cnd - o * g.group); }
                QueryCtx c;
                decode_at<false>(g, b, o, hk * g.group + gi, c);
                if (c.inside) {
                    qo = c.b * g.qs[0] + c.pflat * g.qs[1] + c.h * g.qs[2];
                    ro = c.row;
                    mine_inside = true;
                }
            }
            qoff[tid] = qo;
            orow[tid] = ro;
            my_row = ro;
        }
        if (!__syncthreads_or(mine_inside ? 1 : 0)) continue;   // nothing of this tile is inside its sample
        // the rows' statistics travel together with the rows: one global latency per tile, not two
        float my_lse = 0.f, my_delta = 0.f;
        if (mine_inside) {
            my_lse = lse[my_row];
            my_delta = delta[my_row] - (dlse ? dlse[my_row] : 0.f);
        }
        stage_extra_rows(q, dout, qoff, orow, qt, gt, D, Dv, qstr, vstr, tid);
        if (tid < kExtraTileRows) { rl[tid] = my_lse; rd[tid] = my_delta; }
        __syncthreads();
        // ---- phase 1: S and dP of 16 rows x 8 tokens, then p and ds from the fragments ----
        {
            const int mt = warp & 3, nh = warp >> 2;
            float cs[4] = {0.f, 0.f, 0.f, 0.f}, cd[4] = {0.f, 0.f, 0.f, 0.f};
            const int arow = 16 * mt + lr + 8 * (lm & 1), acol = 8 * (lm >> 1);      // A: rows x depth, row-major
            const int brow = 8 * nh + lr, bcol = 8 * (lm & 1);                       // B(k, token) = toks[token][k]
            const uint32_t aq = shared_addr(qt + arow * qstr + acol), ag = shared_addr(gt + arow * vstr + acol);
            const uint32_t bk = shared_addr(ekt + brow * qstr + bcol), bv = shared_addr(evt + brow * vstr + bcol);
            for (int k = 0; k < D; k += 16) {
                uint32_t a[4], b0, b1;
                ldsm_x4(a, aq + 2 * k);
                ldsm_x2(b0, b1, bk + 2 * k);
                mma_16816<T>(cs, a, b0, b1);
            }
            for (int k = 0; k < Dv; k += 16) {
                uint32_t a[4], b0, b1;
                ldsm_x4(a, ag + 2 * k);
                ldsm_x2(b0, b1, bv + 2 * k);
                mma_16816<T>(cd, a, b0, b1);
            }
            const int tk = 8 * nh + 2 * ft;                    // this lane's two tokens
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {                   // fragment rows fg and fg + 8
                const int r = 16 * mt + fg + 8 * hh;
                const bool live = qoff[r] >= 0;
                const float lr_ = rl[r], dl = rd[r];
                float pj[2], dj[2];
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const bool on = live && tk + j < ne;
                    pj[j] = on ? expf(cs[2 * hh + j] * scale - lr_) : 0.f;
                    dj[j] = on ? pj[j] * (cd[2 * hh + j] - dl) * scale : 0.f;
                }
                *reinterpret_cast<uint32_t*>(pt + r * kPStr + tk) = pack_pair<T>(pj[0], pj[1]);
                *reinterpret_cast<uint32_t*>(dst + r * kPStr + tk) = pack_pair<T>(dj[0], dj[1]);
            }
        }
        __syncthreads();
        // ---- phase 2: warp w owns channels 16w .. 16w+15 of dEk and of dEv ----
        {
            const int arow = lr + 8 * (lm >> 1), acol = 8 * (lm & 1);                // A(token, row) = w[row][token], transposed on load
            const int brow = lr + 8 * (lm & 1), bcol = 16 * warp + 8 * (lm >> 1);    // B(row, channel), transposed on load
#pragma unroll
            for (int k = 0; k < kExtraTileRows; k += 16) {
                uint32_t a[4], bm[4];
                if (16 * warp < D) {
                    ldsm_x4_t(a, shared_addr(dst + (k + arow) * kPStr + acol));
                    ldsm_x4_t(bm, shared_addr(qt + (k + brow) * qstr + bcol));
                    mma_16816<T>(acc_k[0], a, bm[0], bm[1]);
                    mma_16816<T>(acc_k[1], a, bm[2], bm[3]);
                }
                if (16 * warp < Dv) {
                    ldsm_x4_t(a, shared_addr(pt + (k + arow) * kPStr + acol));
                    ldsm_x4_t(bm, shared_addr(gt + (k + brow) * vstr + bcol));
                    mma_16816<T>(acc_v[0], a, bm[0], bm[1]);
                    mma_16816<T>(acc_v[1], a, bm[2], bm[3]);
                }
            }
        }
    }
    // ---- this block's partial sums: [token][D | Dv], through shared memory ----
    __syncthreads();
    float* red = reinterpret_cast<float*>(smem_raw);            // [16][W], over the row tiles
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
        const int ch = 16 * warp + 8 * nt + 2 * ft;
        if (16 * warp < D) {
            red[fg * W + ch] = acc_k[nt][0]; red[fg * W + ch + 1] = acc_k[nt][1];
            red[(fg + 8) * W + ch] = acc_k[nt][2]; red[(fg + 8) * W + ch + 1] = acc_k[nt][3];
        }
        if (16 * warp < Dv) {
            red[fg * W + D + ch] = acc_v[nt][0]; red[fg * W + D + ch + 1] = acc_v[nt][1];
            red[(fg + 8) * W + D + ch] = acc_v[nt][2]; red[(fg + 8) * W + D + ch + 1] = acc_v[nt][3];
        }
    }
    __syncthreads();
    float* out = partial + ((((long long)b * g.Hkv + hk) * gridDim.x + seg) * kExtraGroup) * W;
    for (int i = tid; i < ne * W; i += 256) out[i] = red[i];
}

inline int extra_segments(const Geo& g) { return (int)((g.otot * g.group + kExtraSegRows - 1) / kExtraSegRows); }

// Fast path for the additional tokens' gradients; returns false when it does not apply.
template <typename T>
bool launch_extra_fast(const Geo& g, const void* q, const void* ek, const void* ev, const void* lse,
                       const void* delta, const void* dout, const void* dlse, void* dek, void* dev,
                       void* partial, cudaStream_t s)
{
    if constexpr (!std::is_same<typename AccOf<T>::type, float>::value) {
        return false;
    } else {
    if (g.D > 128 || g.Dv > 128 || !partial) return false;
    const int nseg = extra_segments(g);
    const int W = g.D + g.Dv;
    const size_t smem = (size_t)kExtraGroup * 2 * W * sizeof(float);
    for (int e0 = 0; e0 < g.n_extra; e0 += kExtraGroup) {
        const int ne = g.n_extra - e0 < kExtraGroup ? g.n_extra - e0 : kExtraGroup;
        const dim3 grid((unsigned)nseg, (unsigned)g.Hkv, (unsigned)g.B);
        const int dmax = g.D > g.Dv ? g.D : g.Dv;
        bool tiled = false;
        if constexpr (sizeof(T) == 2) {
            // rows must be readable 16 bytes at a time
            const bool aligned = g.D % 8 == 0 && g.Dv % 8 == 0 && g.qs[0] % 8 == 0 && g.qs[1] % 8 == 0 && g.qs[2] % 8 == 0 &&
                                 ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(dout)) & 15u) == 0;
            const bool tokens_aligned = ((reinterpret_cast<uintptr_t>(ek) | reinterpret_cast<uintptr_t>(ev)) & 15u) == 0;
            if (aligned && tokens_aligned && g.D % 16 == 0 && g.Dv % 16 == 0) {        // warp-level tensor-core products
                const size_t msmem = (size_t)(kExtraTileRows + kExtraGroup) * (g.D + 8 + g.Dv + 8) * sizeof(T) +
                                     (size_t)2 * kExtraTileRows * (kExtraGroup + 8) * sizeof(T) +
                                     (size_t)kExtraTileRows * 2 * sizeof(float) + (size_t)kExtraTileRows * 2 * sizeof(long long);
                ensure_dynamic_smem((const void*)extra_grad_mma_kernel<T>, 96 * 1024);
                extra_grad_mma_kernel<T><<<grid, 256, msmem, s>>>(g, (const T*)q, (const T*)ek, (const T*)ev, (const float*)lse,
                    (const float*)delta, (const T*)dout, (const float*)dlse, (float*)partial, e0, ne);
                tiled = true;
            } else if (aligned) {
                const size_t tsmem = (size_t)kExtraTileRows * (g.D + 8 + g.Dv + 8) * sizeof(T) + (size_t)kExtraGroup * W * sizeof(float) +
                                     (size_t)kExtraTileRows * (2 * kExtraGroup + 2) * sizeof(float) + (size_t)kExtraTileRows * 2 * sizeof(long long);
                ensure_dynamic_smem((const void*)extra_grad_tile_kernel<T>, 96 * 1024);
                extra_grad_tile_kernel<T><<<grid, 256, tsmem, s>>>(g, (const T*)q, (const T*)ek, (const T*)ev, (const float*)lse,
                    (const float*)delta, (const T*)dout, (const float*)dlse, (float*)partial, e0, ne);
                tiled = true;
            }
        }
        if (tiled) {
        } else if (dmax <= 32)
            extra_grad_partial_kernel<T, 1><<<grid, kWarps * 32, smem, s>>>(g, (const T*)q, (const T*)ek, (const T*)ev,
                (const float*)lse, (const float*)delta, (const T*)dout, (const float*)dlse, (float*)partial, e0, ne);
        else if (dmax <= 64)
            extra_grad_partial_kernel<T, 2><<<grid, kWarps * 32, smem, s>>>(g, (const T*)q, (const T*)ek, (const T*)ev,
                (const float*)lse, (const float*)delta, (const T*)dout, (const float*)dlse, (float*)partial, e0, ne);
        else
            extra_grad_partial_kernel<T, 4><<<grid, kWarps * 32, smem, s>>>(g, (const T*)q, (const T*)ek, (const T*)ev,
                (const float*)lse, (const float*)delta, (const T*)dout, (const float*)dlse, (float*)partial, e0, ne);
        const long long n = (long long)g.B * g.Hkv * ne * W;
        extra_grad_reduce_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, s>>>(g, (const float*)partial, nseg, e0, ne,
                                                                            (T*)dek, (T*)dev);
        g_launches += 2;
    }
    return true;
    }
}

template <typename T>
cudaError_t fused_fwd_t(const Geo& g, const void* q, const void* k, const void* v, const void* ek,
                        const void* ev, void* out, void* lse, cudaStream_t s)
{
    using A = typename AccOf<T>::type;
    const long long rows = (long long)g.B * g.otot * g.Hq;
    if (rows == 0) return cudaSuccess;
    const size_t smem = (size_t)kWarps * g.D * sizeof(A);
    NATTEN_DISPATCH_N(g.Dv, NDV,
        fused_fwd_kernel<T, NDV><<<grid_for(rows), kWarps * 32, smem, s>>>(
            g, (const T*)q, (const T*)k, (const T*)v, (const T*)ek, (const T*)ev, (T*)out, (A*)lse, rows));
    ++g_launches;
    return cudaGetLastError();
}

template <typename T>
cudaError_t fused_bwd_t(const Geo& g, const void* q, const void* k, const void* v, const void* ek,
                        const void* ev, const void* out, const void* lse, const void* dout,
                        const void* dlse, void* dq, void* dk, void* dv, void* dek, void* dev,
                        void* workspace, cudaStream_t s)
{
    using A = typename AccOf<T>::type;
    const long long qrows = (long long)g.B * g.otot * g.Hq;
    const long long krows = (long long)g.B * g.ltot * g.Hkv;
    A* delta = (A*)workspace;
    cudaError_t err;
    bool dq_partial = g.extents != nullptr;
    for (int a = 0; a < g.rank; ++a) dq_partial = dq_partial || g.st[a] != 1;
    if (dq_partial) {
        err = cudaMemsetAsync(dq, 0, sizeof(T) * (size_t)g.B * g.ltot * g.Hq * g.D, s);
        if (err != cudaSuccess) return err;
    }
    if (qrows > 0) {
        delta_kernel<T><<<grid_for(qrows), kWarps * 32, 0, s>>>((const T*)out, (const T*)dout, delta, qrows, g.Dv);
        ++g_launches;
        const size_t smem = (size_t)kWarps * (g.D + g.Dv) * sizeof(A);
        NATTEN_DISPATCH_N(g.D, ND,
            fused_bwd_dq_kernel<T, ND><<<grid_for(qrows), kWarps * 32, smem, s>>>(
                g, (const T*)q, (const T*)k, (const T*)v, (const T*)ek, (const T*)ev, (const A*)lse, delta,
                (const T*)dout, (const A*)dlse, (T*)dq, qrows));
        ++g_launches;
    }
    if (krows > 0) {
        const size_t smem = (size_t)kWarps * (g.D + g.Dv) * sizeof(A);
        const int dmax = g.D > g.Dv ? g.D : g.Dv;
        NATTEN_DISPATCH_N(dmax, ND,
            fused_bwd_dkdv_kernel<T, ND, ND><<<grid_for(krows), kWarps * 32, smem, s>>>(
                g, (const T*)q, (const T*)k, (const T*)v, (const A*)lse, delta, (const T*)dout,
                (const A*)dlse, (T*)dk, (T*)dv, krows));
        ++g_launches;
    }
    if (g.n_extra > 0 && g.B > 0) {
        void* partial = static_cast<unsigned char*>(workspace) + simt_delta_bytes(g, sizeof(A));
        if (!launch_extra_fast<T>(g, q, ek, ev, lse, delta, dout, dlse, dek, dev, partial, s)) {
            const size_t smem = (size_t)(kWarps + 1) * (g.D + g.Dv) * sizeof(A);
            const int dmax = g.D > g.Dv ? g.D : g.Dv;
            const unsigned blocks = (unsigned)((long long)g.B * g.n_extra * g.Hkv);
            NATTEN_DISPATCH_N(dmax, ND,
                fused_bwd_extra_kernel<T, ND, ND><<<blocks, kWarps * 32, smem, s>>>(
                    g, (const T*)q, (const T*)ek, (const T*)ev, (const A*)lse, delta, (const T*)dout,
                    (const A*)dlse, (T*)dek, (T*)dev));
            ++g_launches;
        }
    }
    return cudaGetLastError();
}

template <typename T>
cudaError_t qk_fwd_t(const Geo& g, const void* q, const void* k, void* logits, cudaStream_t s)
{
    using A = typename AccOf<T>::type;
    const long long rows = (long long)g.B * g.otot * g.Hq;
    if (rows == 0) return cudaSuccess;
    if constexpr (sizeof(T) == 2) {
        if (split_vec_ok(g, g.D, {q, k}, {g.qs[0], g.qs[1], g.qs[2], g.ks[0], g.ks[1], g.ks[2]}, g.ks[1])) {
            const size_t smem = (size_t)kWarps * g.ktot * sizeof(int);
            NATTEN_DISPATCH_LPR(g.D, LPR,
                dot_neighbours_vec_kernel<T, LPR><<<grid_for(rows), kWarps * 32, smem, s>>>(
                    g, (const T*)q, g.qs[0], g.qs[1], g.qs[2], 1, g.D, (const T*)k, g.ks[0], g.ks[1], g.ks[2],
                    g.has_scale ? (float)g.scale : 1.f, 1, (T*)logits, rows));
            ++g_launches;
            return cudaGetLastError();
        }
    }
    qk_fwd_kernel<T><<<grid_for(rows), kWarps * 32, (size_t)kWarps * g.D * sizeof(A), s>>>(
        g, (const T*)q, (const T*)k, (T*)logits, rows);
    ++g_launches;
    return cudaGetLastError();
}

template <typename T>
cudaError_t qk_bwd_t(const Geo& g, const void* q, const void* k, const void* dlogits, void* dq, void* dk,
                     cudaStream_t s)
{
    const long long qrows = (long long)g.B * g.otot * g.Hq;
    const long long krows = (long long)g.B * g.ltot * g.Hkv;
    bool partial = false;
    for (int a = 0; a < g.rank; ++a) partial = partial || g.st[a] != 1;
    if (partial && dq) {
        cudaError_t err = cudaMemsetAsync(dq, 0, sizeof(T) * (size_t)g.B * g.ltot * g.Hq * g.D, s);
        if (err != cudaSuccess) return err;
    }
    bool vec = false;
    if constexpr (sizeof(T) == 2)
        vec = split_vec_ok(g, g.D, {q, k, dq, dk}, {g.qs[0], g.qs[1], g.qs[2], g.ks[0], g.ks[1], g.ks[2]}, g.ks[1]);
    if (qrows > 0 && dq) {                        // dq == nullptr: another kernel has produced it
        if (vec) {
            if constexpr (sizeof(T) == 2) {
                const size_t smem = (size_t)kWarps * g.ktot * sizeof(int);
                NATTEN_DISPATCH_LPR(g.D, LPR,
                    sum_neighbours_vec_kernel<T, LPR><<<grid_for(qrows), kWarps * 32, smem, s>>>(
                        g, (const T*)dlogits, (const T*)k, g.ks[0], g.ks[1], g.ks[2], g.D,
                        g.has_scale ? (float)g.scale : 1.f, 1, (T*)dq, qrows));
            }
        } else {
            NATTEN_DISPATCH_N(g.D, ND,
                qk_bwd_dq_kernel<T, ND><<<grid_for(qrows), kWarps * 32, 0, s>>>(
                    g, (const T*)k, (const T*)dlogits, (T*)dq, qrows));
        }
        ++g_launches;
    }
    if (krows > 0 && dk) {
        if (vec) {
            if constexpr (sizeof(T) == 2) {
                NATTEN_DISPATCH_LPR(g.D, LPR,
                    inverse_gather_vec_kernel<T, LPR><<<grid_for(krows), kWarps * 32, 0, s>>>(
                        g, (const T*)dlogits, (const T*)q, g.qs[0], g.qs[1], g.qs[2], 1, g.D,
                        g.has_scale ? (float)g.scale : 1.f, (T*)dk, krows));
            }
        } else {
            NATTEN_DISPATCH_N(g.D, ND,
                inverse_gather_kernel<T, ND><<<grid_for(krows), kWarps * 32, 0, s>>>(
                    g, (const T*)dlogits, (const T*)q, g.qs[0], g.qs[1], g.qs[2], 1, g.D,
                    g.has_scale ? g.scale : 1.0, (T*)dk, krows));
        }
        ++g_launches;
    }
    return cudaGetLastError();
}

template <typename T>
cudaError_t av_fwd_t(const Geo& g, const void* attn, const void* v, void* out, cudaStream_t s)
{
    const long long rows = (long long)g.B * g.otot * g.Hq;
    if (rows == 0) return cudaSuccess;
    if constexpr (sizeof(T) == 2) {
        if (split_vec_ok(g, g.Dv, {v, out}, {g.vs[0], g.vs[1], g.vs[2]}, g.vs[1])) {
            const size_t smem = (size_t)kWarps * g.ktot * sizeof(int);
            NATTEN_DISPATCH_LPR(g.Dv, LPR,
                sum_neighbours_vec_kernel<T, LPR><<<grid_for(rows), kWarps * 32, smem, s>>>(
                    g, (const T*)attn, (const T*)v, g.vs[0], g.vs[1], g.vs[2], g.Dv, 1.f, 0, (T*)out, rows));
            ++g_launches;
            return cudaGetLastError();
        }
    }
    NATTEN_DISPATCH_N(g.Dv, NDV,
        av_fwd_kernel<T, NDV><<<grid_for(rows), kWarps * 32, 0, s>>>(
            g, (const T*)attn, (const T*)v, (T*)out, rows));
    ++g_launches;
    return cudaGetLastError();
}

template <typename T>
cudaError_t av_bwd_t(const Geo& g, const void* attn, const void* v, const void* dout, void* dattn, void* dv,
                     cudaStream_t s)
{
    using A = typename AccOf<T>::type;
    const long long qrows = (long long)g.B * g.otot * g.Hq;
    const long long krows = (long long)g.B * g.ltot * g.Hkv;
    bool vec = false;
    if constexpr (sizeof(T) == 2) vec = split_vec_ok(g, g.Dv, {v, dout, dv}, {g.vs[0], g.vs[1], g.vs[2]}, g.vs[1]);
    if (qrows > 0 && dattn) {                     // dattn == nullptr: another kernel has produced it
        if (vec) {
            if constexpr (sizeof(T) == 2) {
                const size_t smem = (size_t)kWarps * g.ktot * sizeof(int);
                NATTEN_DISPATCH_LPR(g.Dv, LPR,
                    dot_neighbours_vec_kernel<T, LPR><<<grid_for(qrows), kWarps * 32, smem, s>>>(
                        g, (const T*)dout, 0, 0, 0, 0, g.Dv, (const T*)v, g.vs[0], g.vs[1], g.vs[2], 1.f, 0,
                        (T*)dattn, qrows));
            }
        } else {
            av_bwd_dattn_kernel<T><<<grid_for(qrows), kWarps * 32, (size_t)kWarps * g.Dv * sizeof(A), s>>>(
                g, (const T*)v, (const T*)dout, (T*)dattn, qrows);
        }
        ++g_launches;
    }
    if (krows > 0 && dv) {
        if (vec) {
            if constexpr (sizeof(T) == 2) {
                NATTEN_DISPATCH_LPR(g.Dv, LPR,
                    inverse_gather_vec_kernel<T, LPR><<<grid_for(krows), kWarps * 32, 0, s>>>(
                        g, (const T*)attn, (const T*)dout, 0, 0, 0, 0, g.Dv, 1.f, (T*)dv, krows));
            }
        } else {
            NATTEN_DISPATCH_N(g.Dv, ND,
                inverse_gather_kernel<T, ND><<<grid_for(krows), kWarps * 32, 0, s>>>(
                    g, (const T*)attn, (const T*)dout, 0, 0, 0, 0, g.Dv, 1.0, (T*)dv, krows));
        }
        ++g_launches;
    }
    return cudaGetLastError();
}

#define NATTEN_BY_DTYPE(dtype, CALL)                                   \
    switch (dtype) {                                                   \
        case 0: { using T = float; return CALL; }                      \
        case 1: { using T = __half; return CALL; }                     \
        case 2: { using T = __nv_bfloat16; return CALL; }              \
        case 3: { using T = double; return CALL; }                     \
        default: return cudaErrorInvalidValue;                         \
    }

} // namespace

unsigned long long simt_launch_count() { return g_launches; }
void simt_count_launch(int n) { g_launches += n; }

cudaError_t simt_fused_fwd(int dtype, const Geo& g, const void* q, const void* k, const void* v,
                           const void* ek, const void* ev, void* out, void* lse, cudaStream_t s)
{
    NATTEN_BY_DTYPE(dtype, fused_fwd_t<T>(g, q, k, v, ek, ev, out, lse, s));
}

cudaError_t simt_fused_bwd(int dtype, const Geo& g, const void* q, const void* k, const void* v,
                           const void* ek, const void* ev, const void* out, const void* lse,
                           const void* dout, const void* dlse, void* dq, void* dk, void* dv,
                           void* dek, void* dev, void* workspace, cudaStream_t s)
{
    NATTEN_BY_DTYPE(dtype, fused_bwd_t<T>(g, q, k, v, ek, ev, out, lse, dout, dlse, dq, dk, dv, dek, dev,
                                          workspace, s));
}

// Gradients of the additional tokens only (used next to the tensor-core backward, which
// covers dq/dk/dv).  `delta` must already hold rowsum(out*dout) - dlse.
template <typename T>
cudaError_t fused_bwd_extra_t(const Geo& g, const void* q, const void* ek, const void* ev, const void* lse,
                              const void* delta, const void* dout, void* dek, void* dev, void* partial,
                              cudaStream_t s)
{
    using A = typename AccOf<T>::type;
    if (g.n_extra <= 0 || g.B <= 0) return cudaSuccess;
    if (launch_extra_fast<T>(g, q, ek, ev, lse, delta, dout, nullptr, dek, dev, partial, s)) return cudaGetLastError();
    const size_t smem = (size_t)(kWarps + 1) * (g.D + g.Dv) * sizeof(A);
    const int dmax = g.D > g.Dv ? g.D : g.Dv;
    const unsigned blocks = (unsigned)((long long)g.B * g.n_extra * g.Hkv);
    NATTEN_DISPATCH_N(dmax, ND,
        fused_bwd_extra_kernel<T, ND, ND><<<blocks, kWarps * 32, smem, s>>>(
            g, (const T*)q, (const T*)ek, (const T*)ev, (const A*)lse, (const A*)delta, (const T*)dout,
            (const A*)nullptr, (T*)dek, (T*)dev));
    ++g_launches;
    return cudaGetLastError();
}

cudaError_t simt_fused_bwd_extra(int dtype, const Geo& g, const void* q, const void* ek, const void* ev,
                                 const void* lse, const void* delta, const void* dout, void* dek, void* dev,
                                 void* partial, cudaStream_t s)
{
    NATTEN_BY_DTYPE(dtype, fused_bwd_extra_t<T>(g, q, ek, ev, lse, delta, dout, dek, dev, partial, s));
}

size_t simt_delta_bytes(const Geo& g, size_t acc_size)
{
    const size_t bytes = (size_t)g.B * (size_t)g.otot * (size_t)g.Hq * acc_size;
    return (bytes + 255) & ~(size_t)255;
}

size_t simt_extra_partial_bytes(int dtype, const Geo& g)
{
    if (g.n_extra <= 0 || dtype == 3 || g.D > 128 || g.Dv > 128) return 0;
    const size_t bytes = (size_t)g.B * g.Hkv * (size_t)extra_segments(g) * kExtraGroup * (g.D + g.Dv) * sizeof(float);
    return (bytes + 255) & ~(size_t)255;
}

cudaError_t simt_qk_fwd(int dtype, const Geo& g, const void* q, const void* k, void* logits, cudaStream_t s)
{
    NATTEN_BY_DTYPE(dtype, qk_fwd_t<T>(g, q, k, logits, s));
}

cudaError_t simt_qk_bwd(int dtype, const Geo& g, const void* q, const void* k, const void* dlogits,
                        void* dq, void* dk, cudaStream_t s)
{
    NATTEN_BY_DTYPE(dtype, qk_bwd_t<T>(g, q, k, dlogits, dq, dk, s));
}

cudaError_t simt_av_fwd(int dtype, const Geo& g, const void* attn, const void* v, void* out, cudaStream_t s)
{
    NATTEN_BY_DTYPE(dtype, av_fwd_t<T>(g, attn, v, out, s));
}

cudaError_t simt_av_bwd(int dtype, const Geo& g, const void* attn, const void* v, const void* dout,
                        void* dattn, void* dv, cudaStream_t s)
{
    NATTEN_BY_DTYPE(dtype, av_bwd_t<T>(g, attn, v, dout, dattn, dv, s));
}

} // namespace natten
