// Between the down-projections and the attention of a layer that attends through low-rank
// latents: one kernel per step that takes the float32 result of the stacked product
// [query latent (Rq values) | key/value latent (R values)] of every token and
//
//   cq[t,:] = a[t,:]  * rsqrt(mean(a[t,:]^2) + eps) * q_gain        stored dense, model dtype
//   c[t,:]  = b[t,:]  * rsqrt(mean(b[t,:]^2) + eps) * kv_gain       stored in the paged cache
//
// The key/value latent is the only thing such a layer caches: a store of one "head" of R
// values per token, [pages][1][page_size][R], written at position p_t of the token's request.
// Sums of squares and scales are float32.  A layer that reads another layer's latents has
// no second segment (cache NULL).  One CTA per token; the order of a row's additions
// depends on its width alone.
#include "common.cuh"

KLLM_EXPORT_LAST_ERROR(latent)

namespace {

constexpr int kThreads = 256;

template <typename T>
__global__ void __launch_bounds__(kThreads)
latent_norm_append_kernel(T* __restrict__ q_out, const float* __restrict__ proj, int64_t proj_stride,
                          const float* __restrict__ q_gain, const float* __restrict__ kv_gain, float eps,
                          const int* __restrict__ positions, const int* __restrict__ token_req,
                          const int* __restrict__ block_table, int max_blocks, T* __restrict__ cache, int Rq, int R,
                          int page_size) {
    __shared__ float red[32];
    griddep_wait();
    griddep_launch();
    const int t = blockIdx.x;
    const float* a = proj + (int64_t)t * proj_stride;
    float ss = 0.f;
    for (int i = threadIdx.x; i < Rq; i += kThreads) ss += a[i] * a[i];
    ss = block_sum(ss, red);
    float scale = rsqrtf(ss / (float)Rq + eps);
    T* qo = q_out + (int64_t)t * Rq;
    for (int i = threadIdx.x; i < Rq; i += kThreads) qo[i] = from_f32<T>(a[i] * scale * q_gain[i]);

    if (cache == nullptr) return;
    const float* b = a + Rq;
    ss = 0.f;
    for (int i = threadIdx.x; i < R; i += kThreads) ss += b[i] * b[i];
    ss = block_sum(ss, red);
    scale = rsqrtf(ss / (float)R + eps);
    const int p = positions[t];
    const int lp = p / page_size, slot = p - lp * page_size;
    const int64_t page = block_table[(int64_t)token_req[t] * max_blocks + lp];
    if (page < 0) return;                                   // a table without a page here: checked on the host
    T* row = cache + (page * page_size + slot) * R;
    for (int i = threadIdx.x; i < R; i += kThreads) row[i] = from_f32<T>(b[i] * scale * kv_gain[i]);
}

// The same step for a layer whose queries come straight from the input and whose keys have, beside
// the latent, one rotated part that all heads share.  proj float32 holds per token
// [H heads of (dk plain | dr rotated) query values | R latent values | dr rotated key values].
//
//   q_plain[t, h, :]          = the dk plain query values (model dtype; they are carried into the
//                               latent space by a product per head afterwards)
//   q_full[t, h, R : R + dr]  = the rotated query part, the tail of the query row that meets the
//                               cached row; the head of that row, R values, is left to the caller
//   cache row of t            = [ b * rsqrt(mean(b^2) + eps) * gain  |  rotated key part ]
//
// Pair (i, i + dr / 2) turns by the angle p * freq[i], formed in double precision; cos and sin are
// multiplied by `amplitude`.  The norm's sum and scale and the rotation are float32.
template <typename T>
__global__ void __launch_bounds__(kThreads)
latent_rope_append_kernel(T* __restrict__ q_plain, T* __restrict__ q_full, const float* __restrict__ proj,
                          int64_t proj_stride, const float* __restrict__ kv_gain, float eps,
                          const double* __restrict__ freq, float amplitude, const int* __restrict__ positions,
                          const int* __restrict__ token_req, const int* __restrict__ block_table, int max_blocks,
                          T* __restrict__ cache, int H, int dk, int dr, int R, int page_size) {
    __shared__ float red[32];
    __shared__ float cs[512];
    griddep_wait();
    griddep_launch();
    const int t = blockIdx.x, p = positions[t], half = dr >> 1;
    for (int i = threadIdx.x; i < half; i += kThreads) {
        double s, c;
        sincos((double)p * freq[i], &s, &c);
        cs[i] = (float)c * amplitude;
        cs[half + i] = (float)s * amplitude;
    }
    __syncthreads();
    const float* a = proj + (int64_t)t * proj_stride;
    T* qp = q_plain + (int64_t)t * H * dk;
    for (int e = threadIdx.x; e < H * dk; e += kThreads) {
        const int h = e / dk, i = e - h * dk;
        qp[e] = from_f32<T>(a[h * (dk + dr) + i]);
    }
    T* qf = q_full + (int64_t)t * H * (R + dr);
    for (int e = threadIdx.x; e < H * half; e += kThreads) {
        const int h = e / half, j = e - h * half;
        const float u = a[h * (dk + dr) + dk + j], v = a[h * (dk + dr) + dk + half + j];
        qf[h * (R + dr) + R + j] = from_f32<T>(u * cs[j] - v * cs[half + j]);
        qf[h * (R + dr) + R + half + j] = from_f32<T>(v * cs[j] + u * cs[half + j]);
    }
    if (cache == nullptr) return;
    const float* b = a + (int64_t)H * (dk + dr);
    float ss = 0.f;
    for (int i = threadIdx.x; i < R; i += kThreads) ss += b[i] * b[i];
    ss = block_sum(ss, red);
    const float scale = rsqrtf(ss / (float)R + eps);
    const int lp = p / page_size, slot = p - lp * page_size;
    const int64_t page = block_table[(int64_t)token_req[t] * max_blocks + lp];
    if (page < 0) return;                                   // a table without a page here: checked on the host
    T* row = cache + (page * page_size + slot) * (R + dr);
    for (int i = threadIdx.x; i < R; i += kThreads) row[i] = from_f32<T>(b[i] * scale * kv_gain[i]);
    for (int j = threadIdx.x; j < half; j += kThreads) {
        const float u = b[R + j], v = b[R + half + j];
        row[R + j] = from_f32<T>(u * cs[j] - v * cs[half + j]);
        row[R + half + j] = from_f32<T>(v * cs[j] + u * cs[half + j]);
    }
}

}  // namespace

// proj float32 [n][Rq (+ R)] at row stride proj_stride; q_out [n][Rq] contiguous in the element
// type `dtype`, which is also the cache's.  cache NULL: proj holds the query latents alone.
extern "C" int kllm_latent_norm_append(void* q_out, const float* proj, int64_t proj_stride, const float* q_gain,
                                       const float* kv_gain, float eps, const int* positions, const int* token_req,
                                       const int* block_table, int max_blocks, void* cache, int n, int Rq, int R,
                                       int page_size, int dtype, void* stream) {
    if (n <= 0) return 0;
    if (Rq <= 0 || (cache && R <= 0)) KLLM_FAIL("latent norm: latent sizes %d and %d", Rq, R);
    if (cache && (page_size <= 0 || !block_table || !kv_gain)) KLLM_FAIL("latent norm: cache without pages, table or gain");
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == KLLM_F32)
        kllm_launch((latent_norm_append_kernel<float>), dim3(n), dim3(kThreads), 0, s, (float*)q_out, proj, proj_stride,
                    q_gain, kv_gain, eps, positions, token_req, block_table, max_blocks, (float*)cache, Rq, R, page_size);
    else if (dtype == KLLM_BF16)
        kllm_launch((latent_norm_append_kernel<bf16>), dim3(n), dim3(kThreads), 0, s, (bf16*)q_out, proj, proj_stride,
                    q_gain, kv_gain, eps, positions, token_req, block_table, max_blocks, (bf16*)cache, Rq, R, page_size);
    else
        KLLM_FAIL("latent norm: unknown element type %d", dtype);
    KLLM_LAUNCH_STATUS();
}

// proj float32 [n][H * (dk + dr) + R + dr] at row stride proj_stride; q_plain [n][H * dk] and q_full
// [n][H * (R + dr)] contiguous in the element type `dtype`, which is also the cache's
// [pages][1][page_size][R + dr]; freq double [dr / 2].  cache NULL: the queries alone.
extern "C" int kllm_latent_rope_append(void* q_plain, void* q_full, const float* proj, int64_t proj_stride,
                                       const float* kv_gain, float eps, const double* freq, float amplitude,
                                       const int* positions, const int* token_req, const int* block_table,
                                       int max_blocks, void* cache, int n, int H, int dk, int dr, int R, int page_size,
                                       int dtype, void* stream) {
    if (n <= 0) return 0;
    if (H <= 0 || dk <= 0 || R <= 0 || dr < 0 || (dr & 1) || dr > 512 || (dr > 0 && !freq))
        KLLM_FAIL("latent rope: %d heads of %d + %d over a latent of %d", H, dk, dr, R);
    if (cache && (page_size <= 0 || !block_table || !kv_gain)) KLLM_FAIL("latent rope: cache without pages, table or gain");
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == KLLM_F32)
        kllm_launch((latent_rope_append_kernel<float>), dim3(n), dim3(kThreads), 0, s, (float*)q_plain, (float*)q_full, proj,
                    proj_stride, kv_gain, eps, freq, amplitude, positions, token_req, block_table, max_blocks,
                    (float*)cache, H, dk, dr, R, page_size);
    else if (dtype == KLLM_BF16)
        kllm_launch((latent_rope_append_kernel<bf16>), dim3(n), dim3(kThreads), 0, s, (bf16*)q_plain, (bf16*)q_full, proj,
                    proj_stride, kv_gain, eps, freq, amplitude, positions, token_req, block_table, max_blocks,
                    (bf16*)cache, H, dk, dr, R, page_size);
    else
        KLLM_FAIL("latent rope: unknown element type %d", dtype);
    KLLM_LAUNCH_STATUS();
}
