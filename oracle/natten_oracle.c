/*
 * TEST INFRASTRUCTURE ONLY -- CPU oracle for the neighbourhood-attention path.
 *
 * A plain-C restatement of the reference's pure backend
 * (src/natten_mps/_core/pure.py, src/natten_mps/utils/window.py and the
 * additional-token / varlen wrappers of src/natten_mps/functional.py).  It
 * exists to check the CUDA kernels and to be timed as the CPU baseline; nothing
 * in the shipped package links, imports or falls back to it.
 *
 * Parity pin: tests/golden/ holds outputs of the reference itself (its pure
 * backend, imported unchanged) on seeded inputs; tests/test_oracle_golden.py
 * checks this file against every one of them.
 *
 * Build:  gcc -O3 -fopenmp -fPIC -shared natten_oracle.c -o libnatten_oracle.so -lm
 */
#include <math.h>
#include <stdlib.h>
#include <string.h>

typedef struct {
    int rank;            /* 1, 2 or 3                                           */
    int B, Hq, Hkv, D, Dv;
    int L[3];            /* padded spatial extents                               */
    int K[3], dil[3], stride[3], causal[3];
    int has_scale;       /* split QK only: 0 = return raw dot products          */
    int n_extra;         /* additional key/value tokens per sample               */
    double scale;
    const int* extents;  /* NULL, or [B*rank] per-sample valid extents           */
} ora_params;

typedef struct {
    long long ltot, otot;
    int O[3];
    int ktot;
} ora_geom;

/* Window start of a non-causal axis.  Literal restatement of
 * utils/window.py:91-111 (get_window_start).                                   */
int ora_window_start(int index, int length, int kernel_size, int dilation)
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

/* First bias-table entry of a position's window on one axis.  Literal restatement of
 * utils/window.py:119-135 (get_pb_start); slot kk reads entry ora_pb_start(...) + kk.      */
int ora_pb_start(int index, int length, int kernel_size, int dilation)
{
    const int nh = kernel_size / 2;
    if (dilation <= 1) {
        int pb = nh;
        if (index < nh) pb += nh - index;
        else if (index + nh >= length) pb += length - index - 1 - nh;
        return pb;
    }
    if (index - nh * dilation < 0) return kernel_size - 1 - index / dilation;
    if (index + nh * dilation >= length) return (length - index - 1) / dilation;
    return nh;
}

/* Key position of slot kk on one axis, or -1 when the slot is masked.
 * Non-causal: start + kk*dilation (_core/pure.py:27-41).  Causal:
 * p - (K-1-kk)*dilation, valid iff >= 0 (_core/pure.py:44-56).  A position
 * outside [0, L) (reachable only with even kernel sizes) counts as masked.     */
static int ora_axis_key(int p, int L, int K, int dil, int causal, int kk)
{
    int pos;
    if (causal) pos = p - (K - 1 - kk) * dil;
    else pos = ora_window_start(p, L, K, dil) + kk * dil;
    if (pos < 0 || pos >= L) return -1;
    return pos;
}

static void ora_make_geom(const ora_params* P, ora_geom* G)
{
    G->ltot = 1; G->otot = 1; G->ktot = 1;
    for (int a = 0; a < 3; ++a) {
        G->O[a] = 1;
        if (a < P->rank) {
            /* output extent = ceil(L / stride): _core/pure.py:18-24 */
            G->O[a] = (P->L[a] + P->stride[a] - 1) / P->stride[a];
            G->ltot *= P->L[a];
            G->otot *= G->O[a];
            G->ktot *= P->K[a];
        }
    }
}

static void ora_sample_extents(const ora_params* P, int b, int* Ls)
{
    for (int a = 0; a < P->rank; ++a)
        Ls[a] = P->extents ? P->extents[b * P->rank + a] : P->L[a];
}

/* Decode flat output index -> query position per axis (o * stride).  Returns 0
 * when the position lies outside the sample's valid extent.                    */
static int ora_query_pos(const ora_params* P, const ora_geom* G, long long o, const int* Ls, int* pos)
{
    int inside = 1;
    for (int a = P->rank - 1; a >= 0; --a) {
        pos[a] = (int)(o % G->O[a]) * P->stride[a];
        o /= G->O[a];
        if (pos[a] >= Ls[a]) inside = 0;
    }
    return inside;
}

/* Flat key index of every slot in row-major (k0, k1, k2) order, -1 = masked
 * (_core/pure.py:91-129 for 2-D, :335-387 for 3-D).  Addresses use the padded
 * extents; window arithmetic uses the sample's own extents.                    */
static void ora_neighbours_impl(const ora_params* P, const int* pos, const int* Ls, int* idx)
{
    int ax[3][1024];
    for (int a = 0; a < P->rank; ++a)
        for (int kk = 0; kk < P->K[a]; ++kk)
            ax[a][kk] = ora_axis_key(pos[a], Ls[a], P->K[a], P->dil[a], P->causal[a], kk);
    int j = 0;
    if (P->rank == 1) {
        for (int k0 = 0; k0 < P->K[0]; ++k0) idx[j++] = ax[0][k0];
    } else if (P->rank == 2) {
        for (int k0 = 0; k0 < P->K[0]; ++k0)
            for (int k1 = 0; k1 < P->K[1]; ++k1)
                idx[j++] = (ax[0][k0] < 0 || ax[1][k1] < 0) ? -1 : ax[0][k0] * P->L[1] + ax[1][k1];
    } else {
        for (int k0 = 0; k0 < P->K[0]; ++k0)
            for (int k1 = 0; k1 < P->K[1]; ++k1)
                for (int k2 = 0; k2 < P->K[2]; ++k2)
                    idx[j++] = (ax[0][k0] < 0 || ax[1][k1] < 0 || ax[2][k2] < 0)
                                   ? -1
                                   : (ax[0][k0] * P->L[1] + ax[1][k1]) * P->L[2] + ax[2][k2];
    }
}

static long long ora_flat_impl(const ora_params* P, const int* pos)
{
    long long f = 0;
    for (int a = 0; a < P->rank; ++a) f = f * P->L[a] + pos[a];
    return f;
}

#define ora_neighbours(P, G, pos, Ls, idx) ora_neighbours_impl((P), (pos), (Ls), (idx))
#define ora_flat(G, pos) ora_flat_impl(P, (pos))

#define REAL float
#define SUF _f32
#include "natten_oracle_body.inc"
#undef REAL
#undef SUF

#define REAL double
#define SUF _f64
#include "natten_oracle_body.inc"
#undef REAL
#undef SUF
