// C-ABI entry points (include/natten_b200.h): argument checks, geometry set-up
// and dispatch between the tcgen05 kernels and the SIMT kernels.
#include "../../include/natten_b200.h"

#include "rpb.cuh"
#include "simt_kernels.cuh"
#include "tc_kernels.cuh"

#include <cstdint>

namespace natten {
namespace {

thread_local int t_last_path = NATTEN_PATH_NONE;

size_t elem_size(int dtype)
{
    switch (dtype) {
        case NATTEN_F32: return 4;
        case NATTEN_F16: case NATTEN_BF16: return 2;
        case NATTEN_F64: return 8;
    }
    return 0;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Validate and expand the caller's params.  `need_qk`: the op uses q/k (and dim).
int make_geo(const natten_params_t* p, Geo& g)
{
    if (!p) return NATTEN_E_INVALID;
    if (p->rank < 1 || p->rank > 3) return NATTEN_E_INVALID;
    if (elem_size(p->dtype) == 0) return NATTEN_E_INVALID;
    if (p->batch < 0 || p->heads_q <= 0 || p->heads_kv <= 0 || p->dim <= 0 || p->dim_v <= 0)
        return NATTEN_E_INVALID;
    if (p->heads_q % p->heads_kv != 0) return NATTEN_E_INVALID;
    if (p->n_extra < 0) return NATTEN_E_INVALID;
    if (p->dim > 256 || p->dim_v > 256) return NATTEN_E_UNSUPPORTED;
    g.rank = p->rank; g.B = p->batch; g.Hq = p->heads_q; g.Hkv = p->heads_kv;
    g.D = p->dim; g.Dv = p->dim_v; g.group = p->heads_q / p->heads_kv;
    g.ltot = 1; g.otot = 1; g.ktot = 1;
    for (int a = 0; a < 3; ++a) {
        const bool on = a < p->rank;
        g.L[a] = on ? p->extent[a] : 1;
        g.K[a] = on ? p->kernel[a] : 1;
        g.dil[a] = on ? p->dilation[a] : 1;
        g.st[a] = on ? p->stride[a] : 1;
        g.causal[a] = on ? (p->causal[a] != 0) : 0;
        if (g.L[a] <= 0 || g.K[a] <= 0 || g.dil[a] <= 0 || g.st[a] <= 0) return NATTEN_E_INVALID;
        // same bounds as utils/params.py:46-82 of the reference
        if (g.K[a] > g.L[a] || (long long)g.K[a] * g.dil[a] > g.L[a]) return NATTEN_E_INVALID;
        g.O[a] = (g.L[a] + g.st[a] - 1) / g.st[a];
        g.ltot *= g.L[a]; g.otot *= g.O[a];
        if ((long long)g.ktot * g.K[a] > (1 << 20)) return NATTEN_E_UNSUPPORTED;
        g.ktot *= g.K[a];
    }
    g.n_extra = p->n_extra; g.has_scale = p->has_scale; g.scale = p->scale;
    for (int i = 0; i < 3; ++i) { g.qs[i] = p->q_stride[i]; g.ks[i] = p->k_stride[i]; g.vs[i] = p->v_stride[i]; }
    g.extents = p->extents;
    g.vec_ok = 0;
    return NATTEN_OK;
}

// 16-byte row loads are legal when every row start is 16-byte aligned.
void set_vec_ok(Geo& g, int dtype, bool use_q, bool use_k, bool use_v, std::initializer_list<const void*> ptrs)
{
    const long long V = 16 / (long long)elem_size(dtype);
    bool ok = true;
    for (const void* p : ptrs) ok = ok && (p == nullptr || aligned16(p));
    if (use_q || use_k) ok = ok && g.D % V == 0;
    if (use_v) ok = ok && g.Dv % V == 0;
    for (int i = 0; i < 3; ++i) {
        if (use_q) ok = ok && g.qs[i] % V == 0;
        if (use_k) ok = ok && g.ks[i] % V == 0;
        if (use_v) ok = ok && g.vs[i] % V == 0;
    }
    g.vec_ok = ok ? 1 : 0;
}

int from_cuda(cudaError_t e) { return e == cudaSuccess ? NATTEN_OK : (int)e; }

} // namespace
} // namespace natten

using namespace natten;

extern "C" {

int natten_fused_fwd(const natten_params_t* p, const void* q, const void* k, const void* v,
                     const void* extra_k, const void* extra_v, void* out, void* lse, void* stream)
{
    Geo g;
    int rc = make_geo(p, g);
    if (rc) return rc;
    if (!q || !k || !v || !out || !lse) return g.B == 0 ? NATTEN_OK : NATTEN_E_INVALID;
    if (g.n_extra > 0 && (!extra_k || !extra_v)) return NATTEN_E_INVALID;
    set_vec_ok(g, p->dtype, true, true, true, {q, k, v, extra_k, extra_v});
    cudaStream_t s = (cudaStream_t)stream;
    if (!(p->flags & NATTEN_FLAG_FORCE_SIMT)) {
        // small persistent CTAs (four per SM up to head dim 64, two above)
        rc = tc_fused_fwd_small(p->dtype, g, q, k, v, extra_k, extra_v, out, lse, s);
        if (rc != NATTEN_E_UNSUPPORTED) { t_last_path = NATTEN_PATH_TCGEN05; return rc; }
    }
    if (p->flags & NATTEN_FLAG_FORCE_TC) return NATTEN_E_UNSUPPORTED;
    t_last_path = NATTEN_PATH_SIMT;
    return from_cuda(simt_fused_fwd(p->dtype, g, q, k, v, extra_k, extra_v, out, lse, s));
}

size_t natten_workspace_bytes(const natten_params_t* p, int op)
{
    Geo g;
    if (make_geo(p, g)) return 0;
    if (op == NATTEN_OP_FUSED_BWD) {
        // delta = rowsum(out * dout), one accumulator per (batch, query, head); then the
        // partial sums of the additional tokens' gradients
        size_t bytes = simt_delta_bytes(g, p->dtype == NATTEN_F64 ? 8 : 4);
        bytes += simt_extra_partial_bytes(p->dtype, g);
        bytes += tc_bwd_workspace_bytes(p->dtype, g);
        return (bytes + 255) & ~(size_t)255;
    }
    return 0;
}

int natten_fused_bwd(const natten_params_t* p, const void* q, const void* k, const void* v,
                     const void* extra_k, const void* extra_v, const void* out, const void* lse,
                     const void* dout, const void* dlse, void* dq, void* dk, void* dv,
                     void* dextra_k, void* dextra_v, void* workspace, size_t workspace_bytes,
                     void* stream)
{
    Geo g;
    int rc = make_geo(p, g);
    if (rc) return rc;
    if (g.B == 0) return NATTEN_OK;
    if (!q || !k || !v || !out || !lse || !dout || !dq || !dk || !dv) return NATTEN_E_INVALID;
    if (g.n_extra > 0 && (!extra_k || !extra_v || !dextra_k || !dextra_v)) return NATTEN_E_INVALID;
    if (!workspace || workspace_bytes < natten_workspace_bytes(p, NATTEN_OP_FUSED_BWD)) return NATTEN_E_WORKSPACE;
    set_vec_ok(g, p->dtype, true, true, true, {q, k, v, extra_k, extra_v, dout});
    cudaStream_t s = (cudaStream_t)stream;
    if (!(p->flags & NATTEN_FLAG_FORCE_SIMT)) {
        rc = tc_fused_bwd(p->dtype, g, q, k, v, extra_k, extra_v, out, lse, dout, dlse, dq, dk, dv,
                          dextra_k, dextra_v, workspace, s);
        if (rc != NATTEN_E_UNSUPPORTED) { t_last_path = NATTEN_PATH_TCGEN05; return rc; }
    }
    if (p->flags & NATTEN_FLAG_FORCE_TC) return NATTEN_E_UNSUPPORTED;
    t_last_path = NATTEN_PATH_SIMT;
    return from_cuda(simt_fused_bwd(p->dtype, g, q, k, v, extra_k, extra_v, out, lse, dout, dlse, dq, dk,
                                    dv, dextra_k, dextra_v, workspace, s));
}

int natten_qk_fwd(const natten_params_t* p, const void* q, const void* k, void* logits, void* stream)
{
    Geo g;
    int rc = make_geo(p, g);
    if (rc) return rc;
    if (g.B == 0) return NATTEN_OK;
    if (!q || !k || !logits || g.extents || g.n_extra) return NATTEN_E_INVALID;
    set_vec_ok(g, p->dtype, true, true, false, {q, k});
    if (!(p->flags & NATTEN_FLAG_FORCE_SIMT)) {
        rc = tc_scores(p->dtype, g, q, g.qs, k, g.ks, g.has_scale ? (float)g.scale : 1.f, true, logits,
                       (cudaStream_t)stream);
        if (rc == 0) { t_last_path = NATTEN_PATH_TCGEN05; return NATTEN_OK; }
        if (rc > 0) return rc;
        if (p->flags & NATTEN_FLAG_FORCE_TC) return NATTEN_E_UNSUPPORTED;
    }
    t_last_path = NATTEN_PATH_SIMT;
    return from_cuda(simt_qk_fwd(p->dtype, g, q, k, logits, (cudaStream_t)stream));
}

int natten_qk_bwd(const natten_params_t* p, const void* q, const void* k, const void* dlogits,
                  void* dq, void* dk, void* stream)
{
    Geo g;
    int rc = make_geo(p, g);
    if (rc) return rc;
    if (g.B == 0) return NATTEN_OK;
    if (!q || !k || !dlogits || !dq || !dk || g.extents || g.n_extra) return NATTEN_E_INVALID;
    t_last_path = NATTEN_PATH_SIMT;
    // dq[row] = scale * sum_slot dlogits[row, slot] * k[key of slot] is the apply product; dK gathers
    // dlogits * q over the inverse neighbourhood.  Whatever the tensor-core kernels do not cover goes to SIMT.
    bool dq_done = false, dk_done = false;
    if (!(p->flags & NATTEN_FLAG_FORCE_SIMT)) {
        const float sc = g.has_scale ? (float)g.scale : 1.f;
        rc = tc_apply(p->dtype, g, dlogits, k, g.ks, sc, true, dq, (cudaStream_t)stream);
        if (rc > 0) return rc;
        dq_done = rc == 0;
        rc = tc_gather(p->dtype, g, dlogits, q, g.qs, sc, dk, (cudaStream_t)stream);
        if (rc > 0) return rc;
        dk_done = rc == 0;
        if (dq_done || dk_done) t_last_path = NATTEN_PATH_TCGEN05;
        if ((p->flags & NATTEN_FLAG_FORCE_TC) && !(dq_done && dk_done)) return NATTEN_E_UNSUPPORTED;
        if (dq_done && dk_done) return NATTEN_OK;
    }
    return from_cuda(simt_qk_bwd(p->dtype, g, q, k, dlogits, dq_done ? nullptr : dq, dk_done ? nullptr : dk,
                                 (cudaStream_t)stream));
}

int natten_qk_rpb_fwd(const natten_params_t* p, const void* q, const void* k, const void* rpb, void* logits,
                      void* stream)
{
    if (!rpb) return NATTEN_E_INVALID;
    Geo g;
    int rc = make_geo(p, g);
    if (rc) return rc;
    if (g.B == 0) return NATTEN_OK;
    // tensor-core kernel: the bias is added while the logits tile is written out (one pass over the logits)
    if (q && k && logits && !g.extents && !g.n_extra && !(p->flags & NATTEN_FLAG_FORCE_SIMT)) {
        rc = tc_scores(p->dtype, g, q, g.qs, k, g.ks, g.has_scale ? (float)g.scale : 1.f, true, logits,
                       (cudaStream_t)stream, rpb);
        if (rc == 0) { t_last_path = NATTEN_PATH_TCGEN05; return NATTEN_OK; }
        if (rc > 0) return rc;
    }
    // otherwise the logits first, then the bias in a second pass
    rc = natten_qk_fwd(p, q, k, logits, stream);
    if (rc) return rc;
    simt_count_launch(1);
    return rpb_add(p->dtype, g, rpb, logits, (cudaStream_t)stream);
}

int natten_qk_rpb_bwd(const natten_params_t* p, const void* q, const void* k, const void* dlogits,
                      void* dq, void* dk, void* drpb, void* stream)
{
    if (!drpb) return NATTEN_E_INVALID;
    int rc = natten_qk_bwd(p, q, k, dlogits, dq, dk, stream);
    if (rc) return rc;
    Geo g;
    rc = make_geo(p, g);
    if (rc) return rc;
    simt_count_launch(1);
    return rpb_grad(p->dtype, g, dlogits, drpb, (cudaStream_t)stream);
}

int natten_av_fwd(const natten_params_t* p, const void* attn, const void* v, void* out, void* stream)
{
    Geo g;
    int rc = make_geo(p, g);
    if (rc) return rc;
    if (g.B == 0) return NATTEN_OK;
    if (!attn || !v || !out || g.extents || g.n_extra) return NATTEN_E_INVALID;
    if (!(p->flags & NATTEN_FLAG_FORCE_SIMT)) {
        Geo gv = g;
        gv.D = g.Dv;
        rc = tc_apply(p->dtype, gv, attn, v, g.vs, 1.f, false, out, (cudaStream_t)stream);
        if (rc == 0) { t_last_path = NATTEN_PATH_TCGEN05; return NATTEN_OK; }
        if (rc > 0) return rc;
        if (p->flags & NATTEN_FLAG_FORCE_TC) return NATTEN_E_UNSUPPORTED;
    }
    t_last_path = NATTEN_PATH_SIMT;
    return from_cuda(simt_av_fwd(p->dtype, g, attn, v, out, (cudaStream_t)stream));
}

int natten_av_bwd(const natten_params_t* p, const void* attn, const void* v, const void* dout,
                  void* dattn, void* dv, void* stream)
{
    Geo g;
    int rc = make_geo(p, g);
    if (rc) return rc;
    if (g.B == 0) return NATTEN_OK;
    if (!attn || !v || !dout || !dattn || !dv || g.extents || g.n_extra) return NATTEN_E_INVALID;
    set_vec_ok(g, p->dtype, false, false, true, {v, dout});
    t_last_path = NATTEN_PATH_SIMT;
    // d attn[row, slot] = <dout[row], v[key of slot]> is the scores product with x = dout (contiguous rows,
    // indexed by position when the stride is 1); dV gathers attn * dout over the inverse neighbourhood.
    bool da_done = false, dv_done = false;
    bool unit_stride = true;
    for (int a = 0; a < g.rank; ++a) unit_stride = unit_stride && g.st[a] == 1;
    if (!(p->flags & NATTEN_FLAG_FORCE_SIMT) && unit_stride) {
        Geo gv = g;
        gv.D = g.Dv;
        const long long dos[3] = {g.otot * (long long)g.Hq * g.Dv, (long long)g.Hq * g.Dv, g.Dv};
        rc = tc_scores(p->dtype, gv, dout, dos, v, g.vs, 1.f, false, dattn, (cudaStream_t)stream);
        if (rc > 0) return rc;
        da_done = rc == 0;
        rc = tc_gather(p->dtype, gv, attn, dout, dos, 1.f, dv, (cudaStream_t)stream);
        if (rc > 0) return rc;
        dv_done = rc == 0;
        if (da_done || dv_done) t_last_path = NATTEN_PATH_TCGEN05;
        if (da_done && dv_done) return NATTEN_OK;
    }
    if ((p->flags & NATTEN_FLAG_FORCE_TC) && !(da_done && dv_done)) return NATTEN_E_UNSUPPORTED;
    return from_cuda(simt_av_bwd(p->dtype, g, attn, v, dout, da_done ? nullptr : dattn, dv_done ? nullptr : dv,
                                 (cudaStream_t)stream));
}

const char* natten_strerror(int code)
{
    switch (code) {
        case NATTEN_OK: return "ok";
        case NATTEN_E_INVALID: return "invalid argument";
        case NATTEN_E_UNSUPPORTED: return "unsupported configuration";
        case NATTEN_E_WORKSPACE: return "workspace missing or too small";
        case NATTEN_E_DEVICE: return "device-side wait timed out";
        case NATTEN_E_TOO_LARGE: return "problem exceeds the built-in scratch of the no-allocation entry point";
    }
    if (code > 0) return cudaGetErrorString((cudaError_t)code);
    return "unknown error";
}

int natten_abi_version(void) { return 1; }
int natten_last_path(void) { return t_last_path; }
unsigned long long natten_launch_count(void) { return simt_launch_count() + tc_launch_count(); }
int natten_device_status(void) { return tc_device_status() == 0 ? NATTEN_OK : NATTEN_E_DEVICE; }
int natten_clear_status(void) { return tc_clear_status(); }
int natten_status_async(int32_t* pinned_host_word, void* stream)
{
    return tc_status_async(reinterpret_cast<int*>(pinned_host_word), (cudaStream_t)stream);
}
void natten_debug_wait(long long budget_cycles, int inject) { tc_debug_wait(budget_cycles, inject); }

} // extern "C"
