// Latent attention: keys and values of all heads are expansions of one normed latent row per token, and one rotated
// key part is shared by the heads, so the cache holds a single row [latent | rotated part] per token.  Because the
// expansions are linear, attention runs over those rows directly: a head's query is carried into the latent space
// (q_lat = Wuk_h^T q_plain), its score is q_lat . latent + q_rot . k_rot, the weighted sum of latent rows comes back
// through the head's value expansion (Wuv_h).  This file holds what stands between the products and the attention
// kernel: the tail of the down product (two norms, rotation, cache write), the tail of the query product (rotation,
// split) and the per-head product that serves both Wuk_h^T and Wuv_h.  Norms, rotation and sums are float32.
#include "attention_common.cuh"

static thread_local cudaError_t g_launch_err = cudaSuccess;      // what the last launch_pdl returned

namespace hfb {
int *error_word();

constexpr int LS_THREADS = 128;          // threads of a block of latent_split_kernel for narrow rows; up to 512 for wide ones
constexpr int LS_MAX_WARPS = 16;

// One block per token: the row [query latent | key/value latent | rotated part] is summed over the product's partial sums
// into shared memory with 16-byte reads (where the sizes allow), both sums of squares are reduced in one go, and the three
// parts leave in their forms: two normed and weighted, one rotated in pairs (2i, 2i + 1).
template <typename TO>
__global__ void __launch_bounds__(LS_MAX_WARPS * 32)
latent_split_kernel(const float *src, int splits, const float *q_w, const float *kv_w, float eps, const float *cos_sin,
                    int n_positions, const int32_t *positions, const int32_t *slots, TO *cq_out, TO *cache,
                    long long cache_slots, int T, int q_rank, int kv_rank, int rot, int *err)
{
    pdl_entry();
    pdl_sync_small();
    extern __shared__ __align__(16) float x[];
    __shared__ float red[2][LS_MAX_WARPS];
    const int threads = blockDim.x, warps = threads >> 5;
    const int t = blockIdx.x;
    const int C = q_rank + kv_rank + rot, kv0 = q_rank, rot0 = q_rank + kv_rank;
    const size_t plane = (size_t)T * C;
    const float *p = src + (size_t)t * C;
    float ss_q = 0.f, ss_kv = 0.f;
    const bool vec = ((q_rank | kv_rank | rot) & 3) == 0 && ((uintptr_t)src & 15) == 0;
    if (vec) {
        for (int c = threadIdx.x * 4; c < C; c += threads * 4) {
            float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int s = 0; s < splits; s++) {
                const float4 g = *(const float4 *)(p + (size_t)s * plane + c);
                a.x += g.x; a.y += g.y; a.z += g.z; a.w += g.w;
            }
            *(float4 *)(x + c) = a;
            // four values never straddle two parts: every part's size is a multiple of four.  Which of the two forms runs
            // depends on the sizes alone, so a row's sums are made in one order whatever the step looks like.
            float q = 0.f;
            q = fmaf(a.x, a.x, q); q = fmaf(a.y, a.y, q); q = fmaf(a.z, a.z, q); q = fmaf(a.w, a.w, q);
            if (c < kv0) ss_q += q;
            else if (c < rot0) ss_kv += q;
        }
    } else {
        for (int c = threadIdx.x; c < C; c += threads) {
            float a = 0.f;
            for (int s = 0; s < splits; s++) a += p[(size_t)s * plane + c];
            x[c] = a;
            if (c < kv0) ss_q = fmaf(a, a, ss_q);
            else if (c < rot0) ss_kv = fmaf(a, a, ss_kv);
        }
    }
    ss_q = warp_sum(ss_q);
    ss_kv = warp_sum(ss_kv);
    if ((threadIdx.x & 31) == 0) { red[0][threadIdx.x >> 5] = ss_q; red[1][threadIdx.x >> 5] = ss_kv; }
    __syncthreads();
    float sum_q = 0.f, sum_kv = 0.f;
    for (int i = 0; i < warps; i++) { sum_q += red[0][i]; sum_kv += red[1][i]; }
    const float r_q = 1.0f / sqrtf(sum_q / (float)q_rank + eps);
    const float r_kv = 1.0f / sqrtf(sum_kv / (float)kv_rank + eps);
    TO *cq = cq_out + (size_t)t * q_rank;
    for (int c = threadIdx.x; c < q_rank; c += threads) cq[c] = from_f32<TO>(x[c] * r_q * q_w[c]);
    if (!slots) return;
    const long long slot = slots[t];
    if (slot < 0) return;
    if (slot >= cache_slots) { if (threadIdx.x == 0) atomicOr(err, HFB_ERR_SLOT); return; }
    TO *row = cache + (size_t)slot * (kv_rank + rot);
    for (int c = threadIdx.x; c < kv_rank; c += threads) row[c] = from_f32<TO>(x[kv0 + c] * r_kv * kv_w[c]);
    if (rot > 0) {
        int pos = positions[t];
        if (pos < 0 || pos >= n_positions) { if (threadIdx.x == 0) atomicOr(err, HFB_ERR_POSITION); pos = 0; }
        const float *cs = cos_sin + (size_t)pos * (rot / 2) * 2;
        for (int i = threadIdx.x; i < rot / 2; i += threads) {
            float lo, hi;
            rope_pair(x[rot0 + 2 * i], x[rot0 + 2 * i + 1], cs[2 * i], cs[2 * i + 1], lo, hi);
            row[kv_rank + 2 * i] = from_f32<TO>(lo);
            row[kv_rank + 2 * i + 1] = from_f32<TO>(hi);
        }
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

// The float32 run takes the kernel above; bfloat16 operands take the same product on the tensor cores (mma.sync.m16n8k16, bfloat16 operands, float32 sums): a block of four warps takes
// 64 tokens x 64 outputs of one head, each warp 16 tokens; pieces of 128 of k pass through shared memory (rows padded by
// 16 bytes, so that the eight rows of an ldmatrix fall into different banks).  MODE 1 is the tail of latent attention's
// query product in one kernel: its A operand is the plain part of the head's query, read as the float32 (partial) sums of
// that product and rounded to bfloat16 on the way into shared memory, and the head's rotated part is rotated and stored
// beside the result (by the blocks of the first output tile), so that neither a rotation kernel nor a buffer of plain
// parts stands between the query product and attention.
constexpr int HM_T = 64, HM_N = 64, HM_K = 128, HM_KP = HM_K + 8;

template <int MODE>
__global__ void __launch_bounds__(128)
headwise_mma_kernel(const __nv_bfloat16 *in, const float *src, int splits, const __nv_bfloat16 *w, __nv_bfloat16 *out, int T,
                    int H, int N, int K, int in_row, int out_row, const float *cos_sin, int n_positions,
                    const int32_t *positions, int rot, int att_col, int *err)
{
    __shared__ __align__(16) __nv_bfloat16 As[HM_T][HM_KP];
    __shared__ __align__(16) __nv_bfloat16 Ws[HM_N][HM_KP];
    const int t0 = blockIdx.x * HM_T, h = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const __nv_bfloat16 *wh = w + (size_t)h * N * K;
    const bool w_vec = (K & 7) == 0 && ((uintptr_t)w & 15) == 0;
    const size_t C = (size_t)H * in_row, plane = (size_t)T * C;          // MODE 1: a row of the product, one partial sum of it
    // A block walks the output tiles gridDim.y apart.  Where all of k fits one piece (the launch then has one block per
    // token tile and head), the tokens' piece is fetched once and stays in shared memory for every output tile.
    const bool a_stays = K <= HM_K;
    bool first_piece = true;
    for (int n0 = blockIdx.y * HM_N; n0 < N; n0 += gridDim.y * HM_N) {
    float acc[8][4];
#pragma unroll
    for (int i = 0; i < 8; i++) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;

    for (int k0 = 0; k0 < K; k0 += HM_K) {
        // the head's weights: they do not depend on the kernel in front, so the first piece is fetched before the wait
        for (int i = threadIdx.x; i < HM_N * (HM_K / 8); i += 128) {
            const int r = i / (HM_K / 8), c = (i % (HM_K / 8)) * 8;
            const int n = n0 + r, k = k0 + c;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (n < N && k < K) {
                if (w_vec) v = *(const uint4 *)(wh + (size_t)n * K + k);
                else {
                    __nv_bfloat16 *e = (__nv_bfloat16 *)&v;
                    for (int j = 0; j < 8 && k + j < K; j++) e[j] = wh[(size_t)n * K + k + j];
                }
            }
            *(uint4 *)&Ws[r][c] = v;
        }
        if (first_piece) pdl_sync();
        const bool fetch_a = first_piece || !a_stays;
        first_piece = false;
        if (!fetch_a) {
        } else if (MODE == 0) {
            const bool a_vec = (in_row & 7) == 0 && (K & 7) == 0 && ((uintptr_t)in & 15) == 0;
            for (int i = threadIdx.x; i < HM_T * (HM_K / 8); i += 128) {
                const int r = i / (HM_K / 8), c = (i % (HM_K / 8)) * 8;
                const int t = t0 + r, k = k0 + c;
                uint4 v = make_uint4(0, 0, 0, 0);
                if (t < T && k < K) {
                    const __nv_bfloat16 *p = in + ((size_t)t * H + h) * in_row + k;
                    if (a_vec) v = *(const uint4 *)p;
                    else {
                        __nv_bfloat16 *e = (__nv_bfloat16 *)&v;
                        for (int j = 0; j < 8 && k + j < K; j++) e[j] = p[j];
                    }
                }
                *(uint4 *)&As[r][c] = v;
            }
        } else {
            const bool a_vec = (in_row & 3) == 0 && (K & 3) == 0 && ((uintptr_t)src & 15) == 0;
#pragma unroll 4
            for (int i = threadIdx.x; i < HM_T * (HM_K / 4); i += 128) {
                const int r = i / (HM_K / 4), c = (i % (HM_K / 4)) * 4;
                const int t = t0 + r, k = k0 + c;
                float4 f = make_float4(0.f, 0.f, 0.f, 0.f);
                if (t < T && k < K) {
                    const float *p = src + (size_t)t * C + (size_t)h * in_row + k;
                    if (a_vec) {
                        for (int sp = 0; sp < splits; sp++) {
                            const float4 g = *(const float4 *)(p + (size_t)sp * plane);
                            f.x += g.x; f.y += g.y; f.z += g.z; f.w += g.w;
                        }
                    } else {
                        float *e = (float *)&f;
                        for (int j = 0; j < 4 && k + j < K; j++)
                            for (int sp = 0; sp < splits; sp++) e[j] += p[(size_t)sp * plane + j];
                    }
                }
                uint2 v;
                v.x = pack_bf16(f.x, f.y);
                v.y = pack_bf16(f.z, f.w);
                *(uint2 *)&As[r][c] = v;
            }
        }
        __syncthreads();
        const int k_here = min(HM_K, K - k0);
        const uint32_t a_base = (uint32_t)__cvta_generic_to_shared(&As[warp * 16 + (lane & 15)][(lane >> 4) * 8]);
        const uint32_t b_base = (uint32_t)__cvta_generic_to_shared(&Ws[(lane & 7) + ((lane >> 4) << 3)][((lane >> 3) & 1) * 8]);
        for (int kk = 0; kk < k_here; kk += 16) {
            uint32_t a[4];
            ldsm_x4(a_base + kk * 2, a[0], a[1], a[2], a[3]);
#pragma unroll
            for (int nn = 0; nn < 8; nn += 2) {
                uint32_t b0, b1, b2, b3;
                ldsm_x4(b_base + (uint32_t)(nn * 8 * HM_KP + kk) * 2, b0, b1, b2, b3);
                mma_bf16(acc[nn], a, b0, b1);
                mma_bf16(acc[nn + 1], a, b2, b3);
            }
        }
        __syncthreads();
    }
    // C fragment: rows lane / 4 and + 8 of the warp's 16 tokens, columns 2 (lane % 4) and + 1 of each group of 8 outputs
    const bool pair_ok = (out_row & 1) == 0 && ((uintptr_t)out & 3) == 0;
#pragma unroll
    for (int half = 0; half < 2; half++) {
        const int t = t0 + warp * 16 + (lane >> 2) + half * 8;
        if (t >= T) continue;
        __nv_bfloat16 *o = out + ((size_t)t * H + h) * out_row;
#pragma unroll
        for (int nn = 0; nn < 8; nn++) {
            const int n = n0 + nn * 8 + (lane & 3) * 2;
            const float x = acc[nn][half * 2], y = acc[nn][half * 2 + 1];
            if (n + 1 < N && pair_ok) *(uint32_t *)(o + n) = pack_bf16(x, y);
            else {
                if (n < N) o[n] = __float2bfloat16_rn(x);
                if (n + 1 < N) o[n + 1] = __float2bfloat16_rn(y);
            }
        }
    }
    }
    if (MODE == 1 && blockIdx.y == 0 && rot > 0) {
        // the head's rotated part: columns K .. K + rot of its piece of the product's row
        const int half_rot = rot / 2;
        for (int i = threadIdx.x; i < HM_T * half_rot; i += 128) {
            const int t = t0 + i / half_rot, j = i % half_rot;
            if (t >= T) break;
            int pos = positions[t];
            if (pos < 0 || pos >= n_positions) { atomicOr(err, HFB_ERR_POSITION); pos = 0; }
            const float *p = src + (size_t)t * C + (size_t)h * in_row + K + 2 * j;
            float a = 0.f, b = 0.f;
            for (int sp = 0; sp < splits; sp++) { a += p[(size_t)sp * plane]; b += p[(size_t)sp * plane + 1]; }
            const float *cs = cos_sin + ((size_t)pos * half_rot + j) * 2;
            float lo, hi;
            rope_pair(a, b, cs[0], cs[1], lo, hi);
            __nv_bfloat16 *o = out + ((size_t)t * H + h) * out_row + att_col + 2 * j;
            o[0] = __float2bfloat16_rn(lo);
            o[1] = __float2bfloat16_rn(hi);
        }
    }
}

}  // namespace hfb

using namespace hfb;

// Blocks per (token tile, head): one that walks all output tiles with the tokens' piece resident, where there are token
// tiles enough to fill the SMs and all of k fits one piece; else one per output tile (few tokens: the blocks only wait for
// their weights, and side by side they wait once).
static int headwise_tiles_y(int T, int N, int K) { return (K <= HM_K && T >= 512) ? 1 : (N + HM_N - 1) / HM_N; }

extern "C" int hfb_latent_split(const float *src, int splits, const float *q_w, const float *kv_w, float eps, const float *cos_sin,
                                int n_positions, const int32_t *positions, const int32_t *slots, void *cq_out, void *cache,
                                int out_dt, int64_t cache_slots, int T, int q_rank, int kv_rank, int rot, hfb_stream s)
{
    if (T <= 0) return HFB_OK;
    if (!valid_dt(out_dt) || splits < 1 || q_rank <= 0 || kv_rank <= 0 || rot < 0 || (rot & 1) || !q_w || !kv_w || !cq_out)
        return fail(HFB_EINVAL, "latent_split: bad arguments (q_rank=%d kv_rank=%d rot=%d)", q_rank, kv_rank, rot);
    if (rot > 0 && (!cos_sin || !positions)) return fail(HFB_EINVAL, "latent_split: rotation needs a table and positions");
    if (slots && !cache) return fail(HFB_EINVAL, "latent_split: the latent rows need a cache");
    const size_t smem = (size_t)(q_rank + kv_rank + rot) * sizeof(float);
    if (smem > 40 * 1024) return fail(HFB_ENOTSUP, "latent_split: rows above %d values are not supported", 40 * 1024 / 4);
    const dim3 grid(T);
    // The number of threads goes with the row's width only, never with the number of tokens: the order in which a row's
    // squares are summed must not depend on what else the step holds.
    const int row = q_rank + kv_rank + rot;
    const dim3 block(row >= 2048 ? LS_MAX_WARPS * 32 : (row >= 768 ? 256 : LS_THREADS));
    if (out_dt == HFB_F32)
        g_launch_err = launch_pdl(latent_split_kernel<float>, grid, block, smem, (cudaStream_t)s, src, splits, q_w, kv_w, eps, cos_sin,
                                  n_positions, positions, slots, (float *)cq_out, (float *)cache, (long long)cache_slots, T, q_rank, kv_rank, rot, error_word());
    else
        g_launch_err = launch_pdl(latent_split_kernel<__nv_bfloat16>, grid, block, smem, (cudaStream_t)s, src, splits, q_w, kv_w, eps, cos_sin,
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
    if (in_dt == HFB_BF16) {
        const dim3 mgrid((T + HM_T - 1) / HM_T, headwise_tiles_y(T, N, K), H);
        g_launch_err = launch_pdl(headwise_mma_kernel<0>, mgrid, dim3(128), 0, (cudaStream_t)s, (const __nv_bfloat16 *)in, (const float *)nullptr, 1,
                                  (const __nv_bfloat16 *)w, (__nv_bfloat16 *)out, T, H, N, K, in_row, out_row, (const float *)nullptr, 0,
                                  (const int32_t *)nullptr, 0, 0, error_word());
        return check_pdl_launch(g_launch_err, "headwise_linear");
    }
    const dim3 grid((T + HW_TT - 1) / HW_TT, (N + HW_NT - 1) / HW_NT, H);
    g_launch_err = launch_pdl(headwise_linear_kernel<float, float, float>, grid, dim3(256), 0, (cudaStream_t)s, (const float *)in, (const float *)w,
                              (float *)out, T, H, N, K, in_row, out_row);
    return check_pdl_launch(g_launch_err, "headwise_linear");
}

extern "C" int hfb_latent_query_absorb(const float *src, int splits, const float *cos_sin, int n_positions, const int32_t *positions,
                                       const void *w_ukt, void *q_att, int T, int H, int d, int rot, int kv_rank, hfb_stream s)
{
    if (T <= 0) return HFB_OK;
    if (splits < 1 || H <= 0 || d <= 0 || kv_rank <= 0 || rot < 0 || (rot & 1) || !src || !w_ukt || !q_att)
        return fail(HFB_EINVAL, "latent_query_absorb: bad arguments (H=%d d=%d rot=%d kv_rank=%d)", H, d, rot, kv_rank);
    if (rot > 0 && (!cos_sin || !positions)) return fail(HFB_EINVAL, "latent_query_absorb: rotation needs a table and positions");
    if (H > 65535) return fail(HFB_ENOTSUP, "latent_query_absorb: sizes exceed the grid limit");
    const dim3 grid((T + HM_T - 1) / HM_T, headwise_tiles_y(T, kv_rank, d), H);
    g_launch_err = launch_pdl(headwise_mma_kernel<1>, grid, dim3(128), 0, (cudaStream_t)s, (const __nv_bfloat16 *)nullptr, src, splits,
                              (const __nv_bfloat16 *)w_ukt, (__nv_bfloat16 *)q_att, T, H, kv_rank, d, d + rot, kv_rank + rot, cos_sin, n_positions,
                              positions, rot, kv_rank, error_word());
    return check_pdl_launch(g_launch_err, "latent_query_absorb");
}
