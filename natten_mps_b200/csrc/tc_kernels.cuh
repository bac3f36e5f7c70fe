// Launchers of the tcgen05 / TMA kernels.  They return NATTEN_E_UNSUPPORTED (-2)
// for configurations they do not cover so that the caller can take the SIMT path.
#pragma once
#include "geometry.cuh"
#include <stddef.h>

namespace natten {

// Fused forward for head dims up to 128 from small persistent CTAs (four per SM up to head dim 64, two above;
// 64-key chunks, interleaved chunk rows).
int tc_fused_fwd_small(int dtype, const Geo& g, const void* q, const void* k, const void* v,
                       const void* ek, const void* ev, void* out, void* lse, cudaStream_t s);
int tc_fused_bwd(int dtype, const Geo& g, const void* q, const void* k, const void* v,
                 const void* ek, const void* ev, const void* out, const void* lse, const void* dout,
                 const void* dlse, void* dq, void* dk, void* dv, void* dek, void* dev,
                 void* workspace, cudaStream_t s);
size_t tc_bwd_workspace_bytes(int dtype, const Geo& g);
// out[row, slot] = scale * <x[row], y[key of slot]> (QK forward; AV backward w.r.t. attn).  x is indexed by
// input position with strides xs (batch, token, head); masked slots get -inf (neg_inf) or 0.
// With `rpb` (a relative position bias table [Hq, 2K-1, ...], unit stride, no causal axis) the bias of every slot is
// added while the finished tile is written out.
int tc_scores(int dtype, const Geo& g, const void* x, const long long xs[3], const void* y, const long long ys[3],
              float scale, bool neg_inf, void* out, cudaStream_t s, const void* rpb = nullptr);
// out[row] = scale * sum_slot w[row, slot] * y[key of slot] (AV forward; QK backward w.r.t. q).
int tc_apply(int dtype, const Geo& g, const void* w, const void* y, const long long ys[3], float scale,
             bool out_by_position, void* out, cudaStream_t s);
// dst[key] = scale * sum over attending (query, head) pairs of w[query, slot] * x[query]  (dK of the QK backward,
// dV of the AV backward); unit stride.
int tc_gather(int dtype, const Geo& g, const void* w, const void* x, const long long xs[3], float scale,
              void* dst, cudaStream_t s);
void tc_count_launch();
unsigned long long tc_launch_count();
// 0 = clean; 1 = some kernel gave up on a bounded wait (synchronises the device).
int tc_device_status();
// Reset the status word of the current device (synchronises); returns a cudaError_t value.
int tc_clear_status();
// Enqueue a copy of the current device's status word into `host_word` (pinned host memory) on stream s.
int tc_status_async(int* host_word, cudaStream_t s);
// Test hooks: cycle budget of the barrier waits (<= 0 restores the default) and a fault to inject
// on the host side of the next launches (0 = none, 1 = the fused forward's first barrier expects
// more bytes than its loads deliver, so that its wait runs out).
void tc_debug_wait(long long budget_cycles, int inject);

} // namespace natten
