// Launchers of the SIMT kernels (simt_kernels.cu).  dtype: 0 f32, 1 f16, 2 bf16, 3 f64.
#pragma once
#include "geometry.cuh"

namespace natten {

cudaError_t simt_fused_fwd(int dtype, const Geo& g, const void* q, const void* k, const void* v,
                           const void* ek, const void* ev, void* out, void* lse, cudaStream_t s);
cudaError_t simt_fused_bwd(int dtype, const Geo& g, const void* q, const void* k, const void* v,
                           const void* ek, const void* ev, const void* out, const void* lse,
                           const void* dout, const void* dlse, void* dq, void* dk, void* dv,
                           void* dek, void* dev, void* workspace, cudaStream_t s);
cudaError_t simt_fused_bwd_extra(int dtype, const Geo& g, const void* q, const void* ek, const void* ev,
                                 const void* lse, const void* delta, const void* dout, void* dek, void* dev,
                                 void* partial, cudaStream_t s);
// Workspace layout of the fused backward: [delta, one accumulator per (batch, query, head)]
// [partial sums of the additional tokens' gradients].
size_t simt_delta_bytes(const Geo& g, size_t acc_size);
size_t simt_extra_partial_bytes(int dtype, const Geo& g);
cudaError_t simt_qk_fwd(int dtype, const Geo& g, const void* q, const void* k, void* logits, cudaStream_t s);
cudaError_t simt_qk_bwd(int dtype, const Geo& g, const void* q, const void* k, const void* dlogits,
                        void* dq, void* dk, cudaStream_t s);
cudaError_t simt_av_fwd(int dtype, const Geo& g, const void* attn, const void* v, void* out, cudaStream_t s);
cudaError_t simt_av_bwd(int dtype, const Geo& g, const void* attn, const void* v, const void* dout,
                        void* dattn, void* dv, cudaStream_t s);
unsigned long long simt_launch_count();
void simt_count_launch(int n);

} // namespace natten
