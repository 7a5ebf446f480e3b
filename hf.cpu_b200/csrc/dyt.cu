// Dynamic Tanh normalisation, y = tanh(alpha * x) * w + b: an element-wise norm that takes no statistics of the
// row.  Three forms: the norm of (chosen) rows; the norm of a sublayer's output added into the float32 residual
// stream; and that with the next sublayer's norm of the new residual in the same pass (what the fused
// sum + residual + RMSNorm tail is to the RMSNorm models).  Also the element-wise activations that are not part
// of a product's epilogue, and the scaling of logits.  All arithmetic in float32, tanhf / expf without fast-math.
#include "common.cuh"

static thread_local cudaError_t g_launch_err = cudaSuccess;      // what the last launch_pdl returned

namespace hfb {

struct DytParams { const void *alpha, *w, *b; int dt; };

__device__ __forceinline__ float dyt_one(const DytParams &p, float alpha, float x, int c)
{
    return tanhf(alpha * x) * load_any(p.w, p.dt, c) + load_any(p.b, p.dt, c);
}

// out[m, c] = dyt(x[rows ? rows[m] : m, c])
template <typename TX>
__global__ void dyt_kernel(const TX *x, const int32_t *rows, DytParams p, void *out, int out_dt, int M, int E)
{
    pdl_entry();
    pdl_sync_small();
    const float alpha = load_any(p.alpha, p.dt, 0);
    const size_t total = (size_t)M * E;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int m = (int)(i / E), c = (int)(i % E);
        const size_t src = (size_t)(rows ? rows[m] : m) * E + c;
        store_any(out, out_dt, i, dyt_one(p, alpha, to_f32(x[src]), c));
    }
}

// residual[m, c] += dyt(y[m, c]); with `next`: out[m, c] = dyt_next(residual[m, c]).  y may come in pieces that this
// pass sums, in this order: `splits` partial sums [splits, M, E] of a product (none: splits = 0), the product's bias, and
// the weighted sum of `top` rows per token, sum_j mix_w[m, j] * mix_y[m * top + j, c] (a routed feed-forward's experts).
template <typename TY>
__global__ void dyt_residual_kernel(const TY *y, int splits, const void *bias, int bias_dt, const float *mix_y,
                                    const float *mix_w, int top, DytParams p, float *residual,
                                    int has_next, DytParams next, void *out, int out_dt, int M, int E)
{
    pdl_entry();
    pdl_sync_small();
    const float alpha = load_any(p.alpha, p.dt, 0);
    const float alpha2 = has_next ? load_any(next.alpha, next.dt, 0) : 0.f;
    const size_t total = (size_t)M * E;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int c = (int)(i % E);
        float v = 0.f;
        for (int s = 0; s < splits; s++) v += to_f32(y[(size_t)s * total + i]);
        if (bias) v += load_any(bias, bias_dt, c);
        if (mix_y) {
            const size_t m = i / E;
            float acc = 0.f;
            for (int j = 0; j < top; j++) acc = fmaf(mix_w[m * top + j], mix_y[(m * top + j) * E + c], acc);
            v += acc;
        }
        const float r = residual[i] + dyt_one(p, alpha, v, c);
        residual[i] = r;
        if (has_next) store_any(out, out_dt, i, dyt_one(next, alpha2, r, c));
    }
}

enum { ACT_SILU = 0, ACT_RELU = 1, ACT_GELU_TANH = 2, ACT_RELU2 = 3, ACT_NONE = 4 };

__device__ __forceinline__ float activate(float z, int act)
{
    switch (act) {
    case ACT_SILU: return z / (1.0f + expf(-z));
    case ACT_RELU: return fmaxf(z, 0.f);
    case ACT_GELU_TANH: return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    case ACT_RELU2: { const float r = fmaxf(z, 0.f); return r * r; }
    default: return z;
    }
}

// out[t, f] = act(g) * u; gate and up fill the two halves of a row of gu or alternate along it
template <typename T>
__global__ void glu_kernel(const T *gu, T *out, int F, size_t total, int interleaved, int act)
{
    pdl_entry();
    pdl_sync_small();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / F;
        const int f = (int)(i % F);
        const float g = to_f32(gu[t * 2 * F + (interleaved ? 2 * f : f)]), u = to_f32(gu[t * 2 * F + (interleaved ? 2 * f + 1 : F + f)]);
        out[i] = from_f32<T>(activate(g, act) * u);
    }
}

template <typename T>
__global__ void act_kernel(const T *x, T *out, size_t total, int act)
{
    pdl_entry();
    pdl_sync_small();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
        out[i] = from_f32<T>(activate(to_f32(x[i]), act));
}

__global__ void scale_kernel(float *x, size_t total, float s)
{
    pdl_entry();
    pdl_sync_small();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) x[i] *= s;
}

static unsigned blocks_for(size_t total)
{
    size_t b = (total + 255) / 256;
    return (unsigned)(b < 1 ? 1 : (b > 148 * 16 ? 148 * 16 : b));
}

}  // namespace hfb

using namespace hfb;

extern "C" int hfb_dyt(const void *x, int x_dt, const int32_t *rows, const void *alpha, const void *w, const void *b,
                       int p_dt, void *out, int out_dt, int M, int E, hfb_stream s)
{
    if (M <= 0) return HFB_OK;
    if (!valid_dt(x_dt) || !valid_dt(p_dt) || !valid_dt(out_dt) || E <= 0 || !alpha || !w || !b)
        return fail(HFB_EINVAL, "dyt: bad arguments");
    DytParams p{alpha, w, b, p_dt};
    const unsigned blocks = blocks_for((size_t)M * E);
    if (x_dt == HFB_F32) g_launch_err = launch_pdl(dyt_kernel<float>, dim3(blocks), dim3(256), 0, (cudaStream_t)s, (const float *)x, rows, p, out, out_dt, M, E);
    else g_launch_err = launch_pdl(dyt_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, (cudaStream_t)s, (const __nv_bfloat16 *)x, rows, p, out, out_dt, M, E);
    return check_pdl_launch(g_launch_err, "dyt");
}

extern "C" int hfb_dyt_residual(const void *y, int y_dt, int splits, const void *bias, int bias_dt, const float *mix_y,
                                const float *mix_w, int top, const void *alpha, const void *w, const void *b, int p_dt,
                                float *residual, const void *alpha2, const void *w2, const void *b2, int p2_dt,
                                void *out, int out_dt, int M, int E, hfb_stream s)
{
    if (M <= 0) return HFB_OK;
    const int has_next = out != nullptr;
    if (!valid_dt(y_dt) || !valid_dt(p_dt) || E <= 0 || !alpha || !w || !b || !residual || splits < 0 || (splits > 0 && !y) ||
        (bias && !valid_dt(bias_dt)) || (mix_y && (!mix_w || top < 1)) || (!mix_y && splits < 1) ||
        (has_next && (!alpha2 || !w2 || !b2 || !valid_dt(p2_dt) || !valid_dt(out_dt))))
        return fail(HFB_EINVAL, "dyt_residual: bad arguments");
    DytParams p{alpha, w, b, p_dt}, n{alpha2, w2, b2, p2_dt};
    const unsigned blocks = blocks_for((size_t)M * E);
    if (y_dt == HFB_F32) g_launch_err = launch_pdl(dyt_residual_kernel<float>, dim3(blocks), dim3(256), 0, (cudaStream_t)s, (const float *)y, splits, bias, bias_dt, mix_y, mix_w, top, p, residual, has_next, n, out, out_dt, M, E);
    else g_launch_err = launch_pdl(dyt_residual_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, (cudaStream_t)s, (const __nv_bfloat16 *)y, splits, bias, bias_dt, mix_y, mix_w, top, p, residual, has_next, n, out, out_dt, M, E);
    return check_pdl_launch(g_launch_err, "dyt_residual");
}

extern "C" int hfb_glu(const void *gu, void *out, int dt, int T, int F, int interleaved, int act, hfb_stream s)
{
    if (T <= 0) return HFB_OK;
    if (!valid_dt(dt) || F <= 0 || act < 0 || act > ACT_NONE) return fail(HFB_EINVAL, "glu: bad arguments");
    const size_t total = (size_t)T * F;
    if (dt == HFB_F32) g_launch_err = launch_pdl(glu_kernel<float>, dim3(blocks_for(total)), dim3(256), 0, (cudaStream_t)s, (const float *)gu, (float *)out, F, total, interleaved, act);
    else g_launch_err = launch_pdl(glu_kernel<__nv_bfloat16>, dim3(blocks_for(total)), dim3(256), 0, (cudaStream_t)s, (const __nv_bfloat16 *)gu, (__nv_bfloat16 *)out, F, total, interleaved, act);
    return check_pdl_launch(g_launch_err, "glu");
}

extern "C" int hfb_act(const void *x, void *out, int dt, int64_t total, int act, hfb_stream s)
{
    if (total <= 0) return HFB_OK;
    if (!valid_dt(dt) || act < 0 || act > ACT_NONE) return fail(HFB_EINVAL, "act: bad arguments");
    if (dt == HFB_F32) g_launch_err = launch_pdl(act_kernel<float>, dim3(blocks_for((size_t)total)), dim3(256), 0, (cudaStream_t)s, (const float *)x, (float *)out, (size_t)total, act);
    else g_launch_err = launch_pdl(act_kernel<__nv_bfloat16>, dim3(blocks_for((size_t)total)), dim3(256), 0, (cudaStream_t)s, (const __nv_bfloat16 *)x, (__nv_bfloat16 *)out, (size_t)total, act);
    return check_pdl_launch(g_launch_err, "act");
}

extern "C" int hfb_scale(float *x, int64_t total, float scale, hfb_stream s)
{
    if (total <= 0) return HFB_OK;
    g_launch_err = launch_pdl(scale_kernel, dim3(blocks_for((size_t)total)), dim3(256), 0, (cudaStream_t)s, x, (size_t)total, scale);
    return check_pdl_launch(g_launch_err, "scale");
}
