// Relative position bias for the split QK operator.
//
//   logits[b, pos, h, slot] += rpb[h, pb(pos_0) + slot_0, pb(pos_1) + slot_1, ...]
//
// with rpb of shape [H, 2*K_0 - 1, (2*K_1 - 1, (2*K_2 - 1))] and pb() the bias window start of the
// reference (src/natten_mps/utils/window.py:119-135; used by src/natten_mps/compat/v014.py:66-183):
// in the interior pb = K/2 and slot j looks at relative offset j - K/2; at the edges the window is
// clamped and pb moves so that the same relative offsets keep the same bias entries.
// The bias is added to the finished logits in one pass over them (masked slots hold -inf and stay
// -inf); its gradient is a fixed-order reduction of dlogits, one block per bias entry, so it is
// bit-reproducible.  Unit stride, non-causal (what the reference's bias operators cover).
#include "rpb.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace natten {
namespace {

__host__ __device__ __forceinline__ int pb_start(int index, int length, int kernel_size, int dilation)
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

template <typename T> struct Acc { using type = float; };
template <> struct Acc<double> { using type = double; };
template <typename T> __device__ __forceinline__ typename Acc<T>::type ld(const T* p) { return (typename Acc<T>::type)(*p); }
template <> __device__ __forceinline__ float ld<__half>(const __half* p) { return __half2float(*p); }
template <> __device__ __forceinline__ float ld<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T, typename A> __device__ __forceinline__ T st(A v) { return (T)v; }
template <> __device__ __forceinline__ __half st<__half, float>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 st<__nv_bfloat16, float>(float v) { return __float2bfloat16_rn(v); }

// Bias index of (position, slot) on every axis -> flat index into one head's bias table.
__device__ __forceinline__ long long bias_index(const Geo& g, long long pos_flat, int slot)
{
    int pos[3] = {0, 0, 0}, sl[3] = {0, 0, 0};
    for (int a = g.rank - 1; a >= 0; --a) {
        pos[a] = (int)(pos_flat % g.L[a]);
        pos_flat /= g.L[a];
        sl[a] = slot % g.K[a];
        slot /= g.K[a];
    }
    long long idx = 0;
    for (int a = 0; a < g.rank; ++a)
        idx = idx * (2 * g.K[a] - 1) + pb_start(pos[a], g.L[a], g.K[a], g.dil[a]) + sl[a];
    return idx;
}

template <typename T>
__global__ void __launch_bounds__(256)
rpb_add_kernel(const __grid_constant__ Geo g, const T* __restrict__ rpb, T* __restrict__ logits, long long total,
               long long table)
{
    using A = typename Acc<T>::type;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int slot = (int)(i % g.ktot);
    const long long row = i / g.ktot;               // (b * ltot + pos) * Hq + h
    const int h = (int)(row % g.Hq);
    const long long pos = (row / g.Hq) % g.ltot;
    const A bias = ld(rpb + h * table + bias_index(g, pos, slot));
    logits[i] = st<T, A>(ld(logits + i) + bias);
}

// One block per (head, bias entry): sums dlogits over every (batch, position) whose window maps a slot
// onto this entry, threads striding over (batch, position) and a tree reduction in a fixed order.
template <typename T>
__global__ void __launch_bounds__(256)
rpb_grad_kernel(const __grid_constant__ Geo g, const T* __restrict__ dlogits, T* __restrict__ drpb, long long table)
{
    using A = typename Acc<T>::type;
    __shared__ A red[256];
    const int h = blockIdx.y;
    long long e = blockIdx.x;
    int want[3] = {0, 0, 0};
    for (int a = g.rank - 1; a >= 0; --a) { want[a] = (int)(e % (2 * g.K[a] - 1)); e /= (2 * g.K[a] - 1); }
    A acc = 0;
    const long long n = (long long)g.B * g.ltot;
    for (long long t = threadIdx.x; t < n; t += blockDim.x) {
        long long p = t % g.ltot;
        const long long b = t / g.ltot;
        int slot = 0;
        bool hit = true;
        int pos[3] = {0, 0, 0};
        for (int a = g.rank - 1; a >= 0; --a) { pos[a] = (int)(p % g.L[a]); p /= g.L[a]; }
        for (int a = 0; a < g.rank; ++a) {
            const int s = want[a] - pb_start(pos[a], g.L[a], g.K[a], g.dil[a]);
            if (s < 0 || s >= g.K[a]) hit = false;
            slot = slot * g.K[a] + s;
        }
        if (hit) {
            acc += ld(dlogits + ((b * g.ltot + t % g.ltot) * g.Hq + h) * g.ktot + slot);
        }
    }
    red[threadIdx.x] = acc;
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1) {
        if ((int)threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o];
        __syncthreads();
    }
    if (threadIdx.x == 0) drpb[h * table + blockIdx.x] = st<T, A>(red[0]);
}

long long table_size(const Geo& g)
{
    long long t = 1;
    for (int a = 0; a < g.rank; ++a) t *= 2 * g.K[a] - 1;
    return t;
}

bool supported(const Geo& g)
{
    for (int a = 0; a < g.rank; ++a)
        if (g.st[a] != 1 || g.causal[a] || (g.K[a] & 1) == 0) return false;     // even kernels index past the table
    return g.extents == nullptr && g.n_extra == 0 && g.Hq == g.Hkv;
}

} // namespace

int rpb_add(int dtype, const Geo& g, const void* rpb, void* logits, cudaStream_t s)
{
    if (!supported(g)) return -2;
    const long long total = (long long)g.B * g.ltot * g.Hq * g.ktot;
    if (total == 0) return 0;
    const long long table = table_size(g);
    const unsigned blocks = (unsigned)((total + 255) / 256);
    switch (dtype) {
        case 0: rpb_add_kernel<float><<<blocks, 256, 0, s>>>(g, (const float*)rpb, (float*)logits, total, table); break;
        case 1: rpb_add_kernel<__half><<<blocks, 256, 0, s>>>(g, (const __half*)rpb, (__half*)logits, total, table); break;
        case 2: rpb_add_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(g, (const __nv_bfloat16*)rpb, (__nv_bfloat16*)logits, total, table); break;
        case 3: rpb_add_kernel<double><<<blocks, 256, 0, s>>>(g, (const double*)rpb, (double*)logits, total, table); break;
        default: return -1;
    }
    const cudaError_t err = cudaGetLastError();
    return err == cudaSuccess ? 0 : (int)err;
}

int rpb_grad(int dtype, const Geo& g, const void* dlogits, void* drpb, cudaStream_t s)
{
    if (!supported(g)) return -2;
    const long long table = table_size(g);
    if (table > 0x7fffffffll || g.Hq > 65535) return -2;
    const dim3 grid((unsigned)table, (unsigned)g.Hq);
    switch (dtype) {
        case 0: rpb_grad_kernel<float><<<grid, 256, 0, s>>>(g, (const float*)dlogits, (float*)drpb, table); break;
        case 1: rpb_grad_kernel<__half><<<grid, 256, 0, s>>>(g, (const __half*)dlogits, (__half*)drpb, table); break;
        case 2: rpb_grad_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(g, (const __nv_bfloat16*)dlogits, (__nv_bfloat16*)drpb, table); break;
        case 3: rpb_grad_kernel<double><<<grid, 256, 0, s>>>(g, (const double*)dlogits, (double*)drpb, table); break;
        default: return -1;
    }
    const cudaError_t err = cudaGetLastError();
    return err == cudaSuccess ? 0 : (int)err;
}

} // namespace natten
