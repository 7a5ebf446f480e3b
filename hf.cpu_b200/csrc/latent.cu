// Latent attention: keys and values of all heads are expansions of one normed latent row per token, and one rotated
// key part is shared by the heads, so the cache holds a single row [latent | rotated part] per token.  Because the
// expansions are linear, attention runs over those rows directly: a head's query is carried into the latent space
// (q_lat = Wuk_h^T q_plain), its score is q_lat . latent + q_rot . k_rot, the weighted sum of latent rows comes back
// through the head's value expansion (Wuv_h).  This file holds what stands between the products and the attention
// kernel: the tail of the down product (two norms, rotation, cache write), the tail of the query product (rotation,
// split) and the per-head product that serves both Wuk_h^T and Wuv_h.  Norms, rotation and sums are float32.
#include "common.cuh"

static thread_local cudaError_t g_launch_err = cudaSuccess;      // what the last launch_pdl returned

namespace hfb {
int *error_word();

constexpr int LS_THREADS = 128;

__device__ __forceinline__ float block_sum_128(float v, float *red)
{
    v = warp_sum(v);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    const float total = red[0] + red[1] + red[2] + red[3];
    __syncthreads();
    return total;
}

// One block per (token, unit): unit 0 the query latent, 1 the key/value latent, 2 the rotated key part.
template <typename TO>
__global__ void __launch_bounds__(LS_THREADS)
latent_split_kernel(const float *src, int splits, const float *q_w, const float *kv_w, float eps, const float *cos_sin,
                    int n_positions, const int32_t *positions, const int32_t *slots, TO *cq_out, TO *cache,
                    long long cache_slots, int T, int q_rank, int kv_rank, int rot, int *err)
{
    pdl_entry();
    pdl_sync_small();
    extern __shared__ float x[];
    __shared__ float red[4];
    const int t = blockIdx.x, unit = blockIdx.y;
    const int C = q_rank + kv_rank + rot;
    const int col0 = unit == 0 ? 0 : (unit == 1 ? q_rank : q_rank + kv_rank);
    const int n = unit == 0 ? q_rank : (unit == 1 ? kv_rank : rot);
    TO *dst;
    if (unit == 0) dst = cq_out + (size_t)t * q_rank;
    else {
        if (!slots) return;
        const long long slot = slots[t];
        if (slot < 0) return;
        if (slot >= cache_slots) { if (threadIdx.x == 0) atomicOr(err, HFB_ERR_SLOT); return; }
        dst = cache + (size_t)slot * (kv_rank + rot) + (unit == 1 ? 0 : kv_rank);
    }
    const size_t plane = (size_t)T * C;
    const float *p = src + (size_t)t * C + col0;
    float ss = 0.f;
    for (int c = threadIdx.x; c < n; c += LS_THREADS) {
        float acc = 0.f;
        for (int s = 0; s < splits; s++) acc += p[(size_t)s * plane + c];
        x[c] = acc;
        ss = fmaf(acc, acc, ss);
    }
    if (unit < 2) {
        ss = block_sum_128(ss, red);
        const float r = 1.0f / sqrtf(ss / (float)n + eps);
        const float *w = unit == 0 ? q_w : kv_w;
        for (int c = threadIdx.x; c < n; c += LS_THREADS) dst[c] = from_f32<TO>(x[c] * r * w[c]);
        return;
    }
    __syncthreads();
    int pos = positions[t];
    if (pos < 0 || pos >= n_positions) { if (threadIdx.x == 0) atomicOr(err, HFB_ERR_POSITION); pos = 0; }
    const float *cs = cos_sin + (size_t)pos * (rot / 2) * 2;
    for (int i = threadIdx.x; i < rot / 2; i += LS_THREADS) {
        float lo, hi;
        rope_pair(x[2 * i], x[2 * i + 1], cs[2 * i], cs[2 * i + 1], lo, hi);
        dst[2 * i] = from_f32<TO>(lo);
        dst[2 * i + 1] = from_f32<TO>(hi);
    }
}

// One warp per (token, head) of the query product's row [H heads of d plain | rot rotated].
template <typename TO>
__global__ void __launch_bounds__(128)
latent_query_rope_kernel(const float *src, int splits, const float *cos_sin, int n_positions, const int32_t *positions,
                         TO *q_plain, TO *q_att, int T, int H, int d, int rot, int att_row, int att_col, int *err)
{
    pdl_entry();
    pdl_sync_small();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * 4 + warp;
    if (item >= (long long)T * H) return;
    const int t = (int)(item / H), h = (int)(item % H);
    const int C = H * (d + rot);
    const size_t plane = (size_t)T * C;
    const float *p = src + (size_t)t * C + (size_t)h * (d + rot);
    TO *qp = q_plain + ((size_t)t * H + h) * d;
    for (int c = lane; c < d; c += 32) {
        float acc = 0.f;
        for (int s = 0; s < splits; s++) acc += p[(size_t)s * plane + c];
        qp[c] = from_f32<TO>(acc);
    }
    int pos = positions[t];
    if (pos < 0 || pos >= n_positions) { if (lane == 0) atomicOr(err, HFB_ERR_POSITION); pos = 0; }
    const float *cs = cos_sin + (size_t)pos * (rot / 2) * 2;
    TO *qa = q_att + ((size_t)t * H + h) * att_row + att_col;
    for (int i = lane; i < rot / 2; i += 32) {
        float a = 0.f, b = 0.f;
        for (int s = 0; s < splits; s++) { a += p[(size_t)s * plane + d + 2 * i]; b += p[(size_t)s * plane + d + 2 * i + 1]; }
        float lo, hi;
        rope_pair(a, b, cs[2 * i], cs[2 * i + 1], lo, hi);
        qa[2 * i] = from_f32<TO>(lo);
        qa[2 * i + 1] = from_f32<TO>(hi);
    }
}

// out[t, h, n] = sum_k w[h, n, k] in[t, h, k].  A block takes HW_TT tokens x HW_NT outputs of one head; pieces of
// HW_KC of k pass through shared memory as float32; every output is one thread's sum in ascending k, so a row's result
// does not depend on which other rows share its block.
constexpr int HW_TT = 16, HW_NT = 64, HW_KC = 32;

template <typename TI, typename TW, typename TO>
__global__ void __launch_bounds__(256)
headwise_linear_kernel(const TI *in, const TW *w, TO *out, int T, int H, int N, int K, int in_row, int out_row)
{
    pdl_sync();
    __shared__ float As[HW_TT][HW_KC + 1];
    __shared__ float Ws[HW_NT][HW_KC + 1];
    const int t0 = blockIdx.x * HW_TT, n0 = blockIdx.y * HW_NT, h = blockIdx.z;
    const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;          // output n0 + tx, tokens t0 + ty * 4 .. + 3
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    const TW *wh = w + (size_t)h * N * K;
    for (int k0 = 0; k0 < K; k0 += HW_KC) {
        for (int i = threadIdx.x; i < HW_TT * HW_KC; i += 256) {
            const int r = i / HW_KC, c = i % HW_KC;
            const int t = t0 + r, k = k0 + c;
            As[r][c] = (t < T && k < K) ? to_f32(in[((size_t)t * H + h) * in_row + k]) : 0.f;
        }
        for (int i = threadIdx.x; i < HW_NT * HW_KC; i += 256) {
            const int r = i / HW_KC, c = i % HW_KC;
            const int n = n0 + r, k = k0 + c;
            Ws[r][c] = (n < N && k < K) ? to_f32(wh[(size_t)n * K + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int c = 0; c < HW_KC; c++) {
            const float wv = Ws[tx][c];
#pragma unroll
            for (int i = 0; i < 4; i++) acc[i] = fmaf(As[ty * 4 + i][c], wv, acc[i]);
        }
        __syncthreads();
    }
    const int n = n0 + tx;
    if (n < N)
        for (int i = 0; i < 4; i++) {
            const int t = t0 + ty * 4 + i;
            if (t < T) out[((size_t)t * H + h) * out_row + n] = from_f32<TO>(acc[i]);
        }
}

}  // namespace hfb

using namespace hfb;

extern "C" int hfb_latent_split(const float *src, int splits, const float *q_w, const float *kv_w, float eps, const float *cos_sin,
                                int n_positions, const int32_t *positions, const int32_t *slots, void *cq_out, void *cache,
                                int out_dt, int64_t cache_slots, int T, int q_rank, int kv_rank, int rot, hfb_stream s)
{
    if (T <= 0) return HFB_OK;
    if (!valid_dt(out_dt) || splits < 1 || q_rank <= 0 || kv_rank <= 0 || rot < 0 || (rot & 1) || !q_w || !kv_w || !cq_out)
        return fail(HFB_EINVAL, "latent_split: bad arguments (q_rank=%d kv_rank=%d rot=%d)", q_rank, kv_rank, rot);
    if (rot > 0 && (!cos_sin || !positions)) return fail(HFB_EINVAL, "latent_split: rotation needs a table and positions");
    if (slots && !cache) return fail(HFB_EINVAL, "latent_split: the latent rows need a cache");
    const int widest = q_rank > kv_rank ? (q_rank > rot ? q_rank : rot) : (kv_rank > rot ? kv_rank : rot);
    const size_t smem = (size_t)widest * sizeof(float);
    if (smem > 48 * 1024) return fail(HFB_ENOTSUP, "latent_split: latents above %d values are not supported", 48 * 1024 / 4);
    const dim3 grid(T, rot > 0 ? 3 : 2);
    if (out_dt == HFB_F32)
        g_launch_err = launch_pdl(latent_split_kernel<float>, grid, dim3(LS_THREADS), smem, (cudaStream_t)s, src, splits, q_w, kv_w, eps, cos_sin,
                                  n_positions, positions, slots, (float *)cq_out, (float *)cache, (long long)cache_slots, T, q_rank, kv_rank, rot, error_word());
    else
        g_launch_err = launch_pdl(latent_split_kernel<__nv_bfloat16>, grid, dim3(LS_THREADS), smem, (cudaStream_t)s, src, splits, q_w, kv_w, eps, cos_sin,
                                  n_positions, positions, slots, (__nv_bfloat16 *)cq_out, (__nv_bfloat16 *)cache, (long long)cache_slots, T, q_rank,
                                  kv_rank, rot, error_word());
    return check_pdl_launch(g_launch_err, "latent_split");
}

extern "C" int hfb_latent_query_rope(const float *src, int splits, const float *cos_sin, int n_positions, const int32_t *positions,
                                     void *q_plain, void *q_att, int out_dt, int T, int H, int d, int rot, int att_row, int att_col,
                                     hfb_stream s)
{
    if (T <= 0) return HFB_OK;
    if (!valid_dt(out_dt) || splits < 1 || H <= 0 || d <= 0 || rot < 0 || (rot & 1) || att_col < 0 || att_col + rot > att_row)
        return fail(HFB_EINVAL, "latent_query_rope: bad arguments (H=%d d=%d rot=%d)", H, d, rot);
    if (rot > 0 && (!cos_sin || !positions)) return fail(HFB_EINVAL, "latent_query_rope: rotation needs a table and positions");
    const long long items = (long long)T * H;
    const unsigned blocks = (unsigned)((items + 3) / 4);
    if (out_dt == HFB_F32)
        g_launch_err = launch_pdl(latent_query_rope_kernel<float>, dim3(blocks), dim3(128), 0, (cudaStream_t)s, src, splits, cos_sin, n_positions, positions,
                                  (float *)q_plain, (float *)q_att, T, H, d, rot, att_row, att_col, error_word());
    else
        g_launch_err = launch_pdl(latent_query_rope_kernel<__nv_bfloat16>, dim3(blocks), dim3(128), 0, (cudaStream_t)s, src, splits, cos_sin, n_positions,
                                  positions, (__nv_bfloat16 *)q_plain, (__nv_bfloat16 *)q_att, T, H, d, rot, att_row, att_col, error_word());
    return check_pdl_launch(g_launch_err, "latent_query_rope");
}

extern "C" int hfb_headwise_linear(const void *in, int in_dt, const void *w, int w_dt, void *out, int out_dt, int T, int H, int N,
                                   int K, int in_row, int out_row, hfb_stream s)
{
    if (T <= 0) return HFB_OK;
    if (!valid_dt(in_dt) || !valid_dt(w_dt) || !valid_dt(out_dt) || H <= 0 || N <= 0 || K <= 0 || in_row < K || out_row < N)
        return fail(HFB_EINVAL, "headwise_linear: bad arguments (H=%d N=%d K=%d)", H, N, K);
    if (H > 65535 || (N + HW_NT - 1) / HW_NT > 65535) return fail(HFB_ENOTSUP, "headwise_linear: sizes exceed the grid limit");
    if (in_dt != out_dt || (in_dt == HFB_F32) != (w_dt == HFB_F32))
        return fail(HFB_ENOTSUP, "headwise_linear: operands are all float32 or all bfloat16");
    const dim3 grid((T + HW_TT - 1) / HW_TT, (N + HW_NT - 1) / HW_NT, H);
    if (in_dt == HFB_F32)
        g_launch_err = launch_pdl(headwise_linear_kernel<float, float, float>, grid, dim3(256), 0, (cudaStream_t)s, (const float *)in, (const float *)w,
                                  (float *)out, T, H, N, K, in_row, out_row);
    else
        g_launch_err = launch_pdl(headwise_linear_kernel<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16>, grid, dim3(256), 0, (cudaStream_t)s,
                                  (const __nv_bfloat16 *)in, (const __nv_bfloat16 *)w, (__nv_bfloat16 *)out, T, H, N, K, in_row, out_row);
    return check_pdl_launch(g_launch_err, "headwise_linear");
}
