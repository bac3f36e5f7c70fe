// Relative position bias of the split QK operator (rpb.cu).  Return 0, -1 (bad dtype),
// -2 (configuration not covered: stride, causal axes, GQA, per-sample extents) or a cudaError_t value.
#pragma once
#include "geometry.cuh"

namespace natten {

// logits[b, pos, h, slot] += rpb[h, bias index of (pos, slot)], in place.
int rpb_add(int dtype, const Geo& g, const void* rpb, void* logits, cudaStream_t s);
// drpb[h, entry] = sum of dlogits over every (batch, position, slot) that reads the entry.
int rpb_grad(int dtype, const Geo& g, const void* dlogits, void* drpb, cudaStream_t s);

} // namespace natten
