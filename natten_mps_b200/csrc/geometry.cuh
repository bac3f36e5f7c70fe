// Neighbourhood geometry shared by every kernel: the integer window arithmetic
// of the reference (src/natten_mps/utils/window.py:91-111 and the causal rule of
// src/natten_mps/_core/pure.py:44-56) plus the inverse neighbourhood (which
// queries attend to a given key), computed in closed form instead of the
// reference's CPU-built CSR tables (src/natten_mps/_core/inverse_maps.py:91-123).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace natten {

struct Geo {
    int rank, B, Hq, Hkv, D, Dv, group;
    int L[3], O[3], K[3], dil[3], st[3], causal[3];
    int ktot, n_extra, has_scale, vec_ok;
    long long ltot, otot;
    long long qs[3], ks[3], vs[3];   // batch, token, head strides (elements)
    const int* extents;              // [B, rank] or nullptr
    double scale;
};

__host__ __device__ __forceinline__ int window_start(int index, int length, int kernel_size, int dilation)
{
    const int nh = kernel_size / 2;
    if (dilation <= 1) {
        int start = index - nh > 0 ? index - nh : 0;
        if (index + nh >= length) start += length - index - nh - 1;
        return start;
    }
    const int start = index - nh * dilation;
    if (start < 0) return index % dilation;
    if (index + nh * dilation >= length) {
        const int imodd = index % dilation;
        const int a = (length / dilation) * dilation;
        const int b = length - a;
        if (imodd < b) return length - b + imodd - 2 * nh * dilation;
        return a + imodd - kernel_size * dilation;
    }
    return start;
}

// First key position of the query's window on one axis.  For a causal axis the
// window is [p-(K-1)*dil, p] with no boundary shift; positions < 0 are masked.
__host__ __device__ __forceinline__ int axis_first_key(int p, int L, int K, int dil, int causal)
{
    return causal ? p - (K - 1) * dil : window_start(p, L, K, dil);
}

// Slot (0..K-1) of key position n in query p's window on one axis, or -1.
__host__ __device__ __forceinline__ int axis_slot(int p, int n, int L, int K, int dil, int causal)
{
    const int first = axis_first_key(p, L, K, dil, causal);
    const int diff = n - first;
    if (diff < 0 || diff % dil != 0) return -1;
    const int slot = diff / dil;
    if (slot >= K) return -1;
    if (n < 0 || n >= L) return -1;
    return slot;
}

// Candidate queries of key n on one axis: positions base + t*dil, t in [0,cnt).
// A superset of the inverse neighbourhood; membership is re-checked exactly
// with axis_slot().  For odd kernels the range is exact: inside the key's
// dilation class (n' = n/dil among L' positions) the attending queries are
// [n' <= K-1 ? 0 : n'-K/2,  n' >= L'-K ? L'-1 : n'+K/2].
__host__ __device__ __forceinline__ void axis_candidates(int n, int L, int K, int dil, int causal,
                                                          int& base, int& cnt)
{
    if (causal) {
        base = n;
        const int room = (L - 1 - n) / dil + 1;
        cnt = room < K ? room : K;
        return;
    }
    const int r = n % dil;
    const int np = n / dil;
    const int Lp = (L - r + dil - 1) / dil;
    int lo, hi;
    if (K & 1) {
        lo = (np <= K - 1) ? 0 : np - K / 2;
        hi = (np >= Lp - K) ? Lp - 1 : np + K / 2;
    } else {
        lo = np - K; hi = np + K;
    }
    if (lo < 0) lo = 0;
    if (hi > Lp - 1) hi = Lp - 1;
    base = r + lo * dil;
    cnt = hi - lo + 1;
}

} // namespace natten
