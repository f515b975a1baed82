// Between the stacked q/k/v projection and the attention of a layer whose queries and keys are
// normed head by head and rotated in part: one kernel per step that takes the float32 result of
// the product, [q heads | k heads | v heads] of every token, and
//
//   adds the projections' biases (optional, float32),
//   divides every query and key head by its root mean square over its dk values and multiplies by
//   a gain [dk] that all heads share (optional),
//   turns the pairs (i, i + rot / 2), i < rot / 2, of every query and key head by the angle
//   p * freq[i] (rotate-half layout; the dims from rot on pass unchanged), cos and sin times
//   `amplitude`,
//   stores the queries dense in the model's element type and writes keys and values into the paged
//   caches [pages][k heads][page_size][dk] and [pages][v heads][page_size][dv] at position p.
//
// The number of value heads is independent of the number of key heads (several key heads may
// attend over one value head).  The angle is formed in double precision from a double frequency,
// once per token and pair, so that it is as exact as a table computed on the host would be; sums
// of squares, scales and the rotation are float32.  One CTA per token, one warp per head; a
// head's sums depend on its size alone.
//
// Second kernel: the combination of the maps of a differential attention.  Every head has two
// attention maps over the same values, a1 and a2; o = a1 - lambda * a2 is divided by its root mean
// square over the head's dv values and multiplied by a constant.
#include "common.cuh"

KLLM_EXPORT_LAST_ERROR(qk_headnorm)

namespace {

constexpr int kWarps = 8, kMaxDk = 512, kMaxRot = 512;

template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
headnorm_rope_append_kernel(T* __restrict__ q_out, const float* __restrict__ qkv, int64_t qkv_stride,
                            const float* __restrict__ bias, const float* __restrict__ q_gain,
                            const float* __restrict__ k_gain, float eps, const double* __restrict__ freq,
                            float amplitude, int rot, const int* __restrict__ positions,
                            const int* __restrict__ token_req, const int* __restrict__ block_table, int max_blocks,
                            T* __restrict__ kcache, T* __restrict__ vcache, int q_heads, int k_heads, int v_heads,
                            int dk, int dv, int page_size) {
    __shared__ float cs[kMaxRot];                 // cos (first half), sin (second half) of this token's angles
    __shared__ float buf[kWarps][kMaxDk];
    griddep_wait();
    griddep_launch();
    const int t = blockIdx.x, p = positions[t], half = rot >> 1;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        double s, c;
        sincos((double)p * freq[i], &s, &c);
        cs[i] = (float)c * amplitude;
        cs[half + i] = (float)s * amplitude;
    }
    __syncthreads();
    int64_t page = -1;
    int slot = 0;
    if (kcache != nullptr) {
        page = block_table[(int64_t)token_req[t] * max_blocks + p / page_size];      // never negative for a validated step
        slot = p % page_size;
    }
    const float* row = qkv + (int64_t)t * qkv_stride;
    const int heads = q_heads + (page >= 0 ? k_heads : 0);
    for (int h = warp; h < heads; h += kWarps) {
        const bool is_q = h < q_heads;
        const float* src = row + (int64_t)h * dk;                   // the key heads follow the query heads
        const float* b = bias ? bias + (int64_t)h * dk : nullptr;
        const float* gain = is_q ? q_gain : k_gain;
        float ss = 0.f;
        for (int i = lane; i < dk; i += 32) {
            const float v = src[i] + (b ? b[i] : 0.f);
            buf[warp][i] = v;
            ss += v * v;
        }
        float scale = 1.f;
        if (gain) scale = rsqrtf(warp_sum(ss) / (float)dk + eps);
        __syncwarp();
        T* dst = is_q ? q_out + ((int64_t)t * q_heads + h) * dk
                      : kcache + ((page * k_heads + (h - q_heads)) * page_size + slot) * dk;
        for (int i = lane; i < dk; i += 32) {
            float v = buf[warp][i] * scale * (gain ? gain[i] : 1.f);
            if (i < rot) {
                const int j = i < half ? i : i - half, o = i < half ? i + half : i - half;
                const float w = buf[warp][o] * scale * (gain ? gain[o] : 1.f);
                v = i < half ? v * cs[j] - w * cs[half + j] : v * cs[j] + w * cs[half + j];
            }
            dst[i] = from_f32<T>(v);
        }
        __syncwarp();
    }
    if (page < 0) return;
    const float* vsrc = row + (int64_t)(q_heads + k_heads) * dk;
    const float* vb = bias ? bias + (int64_t)(q_heads + k_heads) * dk : nullptr;
    for (int idx = threadIdx.x; idx < v_heads * dv; idx += blockDim.x) {
        const int g = idx / dv, i = idx - g * dv;
        vcache[((page * v_heads + g) * page_size + slot) * dv + i] = from_f32<T>(vsrc[idx] + (vb ? vb[idx] : 0.f));
    }
}

// a float32 [n][G][2][gs][dv]: head (g, j) has its two maps at [g][0][j] and [g][1][j];
// out [n][G * gs][dv] in T.  One warp per (token, head).
template <typename T>
__global__ void __launch_bounds__(128)
maps_combine_kernel(T* __restrict__ out, const float* __restrict__ a, int n, int G, int gs, int dv, float lambda,
                    float eps, float post) {
    griddep_wait();
    griddep_launch();
    const int lane = threadIdx.x & 31;
    const int64_t item = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (item >= (int64_t)n * G * gs) return;
    const int H = G * gs;
    const int64_t t = item / H;
    const int h = (int)(item - t * H), g = h / gs, j = h - g * gs;
    const float* a1 = a + ((t * G + g) * 2 * gs + j) * dv;
    const float* a2 = a1 + (int64_t)gs * dv;
    float o[kMaxDk / 32], ss = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxDk / 32; i++) {
        const int d = lane + 32 * i;
        o[i] = d < dv ? a1[d] - lambda * a2[d] : 0.f;
        ss += o[i] * o[i];
    }
    const float scale = rsqrtf(warp_sum(ss) / (float)dv + eps) * post;
    T* orow = out + item * dv;
#pragma unroll
    for (int i = 0; i < kMaxDk / 32; i++) {
        const int d = lane + 32 * i;
        if (d < dv) orow[d] = from_f32<T>(o[i] * scale);
    }
}

}  // namespace

// qkv float32 [n][(q_heads + k_heads) * dk + v_heads * dv] at row stride qkv_stride; bias float32 of
// a row's length or NULL; q_gain / k_gain float32 [dk] or NULL (no norm of that side); freq double
// [rot / 2] (NULL with rot 0: nothing is rotated); q_out [n][q_heads * dk] contiguous in the element
// type `dtype`, which is also the caches'.  kcache NULL: only the queries are produced.
extern "C" int kllm_headnorm_rope_append(void* q_out, const float* qkv, int64_t qkv_stride, const float* bias,
                                         const float* q_gain, const float* k_gain, float eps, const double* freq,
                                         float amplitude, int rot, const int* positions, const int* token_req,
                                         const int* block_table, int max_blocks, void* kcache, void* vcache, int n,
                                         int q_heads, int k_heads, int v_heads, int dk, int dv, int page_size, int dtype,
                                         void* stream) {
    if (n <= 0) return 0;
    if (dk <= 0 || dk > kMaxDk || q_heads <= 0) KLLM_FAIL("head norm: %d query heads of size %d (up to %d)", q_heads, dk, kMaxDk);
    if (rot < 0 || rot > dk || (rot & 1) || rot > kMaxRot || (rot > 0 && !freq))
        KLLM_FAIL("head norm: rotary width %d invalid for head size %d", rot, dk);
    if (kcache && (k_heads <= 0 || v_heads <= 0 || dv <= 0 || page_size <= 0 || !vcache || !block_table || !token_req))
        KLLM_FAIL("head norm: a cache write needs key and value heads, pages and tables");
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == KLLM_F32)
        kllm_launch((headnorm_rope_append_kernel<float>), dim3(n), dim3(kWarps * 32), 0, s, (float*)q_out, qkv, qkv_stride,
                    bias, q_gain, k_gain, eps, freq, amplitude, rot, positions, token_req, block_table, max_blocks,
                    (float*)kcache, (float*)vcache, q_heads, k_heads, v_heads, dk, dv, page_size);
    else if (dtype == KLLM_BF16)
        kllm_launch((headnorm_rope_append_kernel<bf16>), dim3(n), dim3(kWarps * 32), 0, s, (bf16*)q_out, qkv, qkv_stride,
                    bias, q_gain, k_gain, eps, freq, amplitude, rot, positions, token_req, block_table, max_blocks,
                    (bf16*)kcache, (bf16*)vcache, q_heads, k_heads, v_heads, dk, dv, page_size);
    else
        KLLM_FAIL("head norm: unknown element type %d", dtype);
    KLLM_LAUNCH_STATUS();
}

// out [n][G * gs][dv] (element type `dtype`) = (a1 - lambda a2) / rms(a1 - lambda a2) * post, from
// a float32 [n][G][2][gs][dv].
extern "C" int kllm_maps_combine(void* out, const float* a, int n, int G, int gs, int dv, float lambda, float eps,
                                 float post, int dtype, void* stream) {
    if (n <= 0) return 0;
    if (G <= 0 || gs <= 0 || dv <= 0 || dv > kMaxDk) KLLM_FAIL("maps combine: %d x %d heads of %d values (up to %d)", G, gs, dv, kMaxDk);
    cudaStream_t s = (cudaStream_t)stream;
    const int64_t items = (int64_t)n * G * gs;
    const unsigned grid = (unsigned)((items + 3) / 4);
    if (dtype == KLLM_F32)
        kllm_launch((maps_combine_kernel<float>), dim3(grid), dim3(128), 0, s, (float*)out, a, n, G, gs, dv, lambda, eps, post);
    else if (dtype == KLLM_BF16)
        kllm_launch((maps_combine_kernel<bf16>), dim3(grid), dim3(128), 0, s, (bf16*)out, a, n, G, gs, dv, lambda, eps, post);
    else
        KLLM_FAIL("maps combine: unknown element type %d", dtype);
    KLLM_LAUNCH_STATUS();
}
