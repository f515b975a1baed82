// Between the q/k/v projection and attention, for layers that normalise queries and keys
// over the whole projection, with or without a rotation after the norm: one kernel per step that
//
//   q[t,:]  = qp[t,:] * rsqrt(mean over all H * dk values of qp[t,:]^2 + eps) * q_gain * temp(p_t)
//   k[t,:]  = kp[t,:] * rsqrt(mean over all G * dk values of kp[t,:]^2 + eps) * k_gain
//   temp(p) = 1 + coef * ln(floor((p + 1) / every) + 1)         (1 when coef == 0)
//
// then, with rot > 0, turns the pairs (i, i + rot / 2), i < rot / 2, of every query and key head by the
// angle p * freq[i] (the dims from rot on pass unchanged; the angle is formed in double precision),
// stores q in the model's element type for the attention kernel, and writes k and v into
// the pages of the cache at position p_t of the token's request.  The projections come
// in float32 (the product's unrounded result); sums of squares, scales and the
// temperature are float32.  Keys have dk values per head, values dv: the two caches are
// [pages][kv heads][page_size][dk] and [pages][kv heads][page_size][dv].
// One CTA per token; the order of a row's additions depends on its width alone.
#include "common.cuh"

KLLM_EXPORT_LAST_ERROR(qknorm_append)

namespace {

constexpr int kThreads = 256;
constexpr int kMaxRot = 512;

// One normed value of a head at column c, rotated when c lies in the head's first `rot` values.
__device__ __forceinline__ float turned(const float* row, const float* gain, float scale, int base, int c, int rot,
                                        const float* cs) {
    const float a = row[base + c] * scale * gain[base + c];
    if (c >= rot) return a;
    const int half = rot >> 1;
    if (c < half) {
        const float b = row[base + c + half] * scale * gain[base + c + half];
        return a * cs[c] - b * cs[half + c];
    }
    const float b = row[base + c - half] * scale * gain[base + c - half];
    return a * cs[c - half] + b * cs[c];
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
qknorm_append_kernel(T* __restrict__ q_out, const float* __restrict__ qkv, int64_t qkv_stride,
                     const float* __restrict__ q_gain, const float* __restrict__ k_gain, float eps, float coef,
                     int every, const int* __restrict__ positions, const int* __restrict__ token_req,
                     const int* __restrict__ block_table, int max_blocks, T* __restrict__ kcache,
                     T* __restrict__ vcache, int n_heads, int n_kv, int dk, int dv, int page_size, int rot,
                     const double* __restrict__ freq) {
    __shared__ float red[32];
    __shared__ float cs[kMaxRot];          // cos of the rot / 2 angles, then their sin
    griddep_wait();
    griddep_launch();
    const int t = blockIdx.x;
    for (int i = threadIdx.x; i < (rot >> 1); i += kThreads) {
        double sn, c;
        sincos((double)positions[t] * freq[i], &sn, &c);
        cs[i] = (float)c;
        cs[(rot >> 1) + i] = (float)sn;
    }
    const int Q = n_heads * dk, K = n_kv * dk, V = n_kv * dv;
    const float* qp = qkv + (int64_t)t * qkv_stride;
    const float* kp = qp + Q;
    const float* vp = kp + K;
    const int p = positions[t];

    float ss = 0.f;
    for (int i = threadIdx.x; i < Q; i += kThreads) ss += qp[i] * qp[i];
    ss = block_sum(ss, red);
    float scale = rsqrtf(ss / (float)Q + eps);
    if (coef != 0.f) scale *= 1.f + coef * logf((float)((p + 1) / every) + 1.f);
    T* qo = q_out + (int64_t)t * Q;
    if (rot == 0) {
        for (int i = threadIdx.x; i < Q; i += kThreads) qo[i] = from_f32<T>(qp[i] * scale * q_gain[i]);
    } else {
        for (int i = threadIdx.x; i < Q; i += kThreads) {
            const int c = i % dk;
            qo[i] = from_f32<T>(turned(qp, q_gain, scale, i - c, c, rot, cs));
        }
    }

    if (kcache == nullptr) return;
    ss = 0.f;
    for (int i = threadIdx.x; i < K; i += kThreads) ss += kp[i] * kp[i];
    ss = block_sum(ss, red);
    scale = rsqrtf(ss / (float)K + eps);
    const int lp = p / page_size, slot = p - lp * page_size;
    const int64_t page = block_table[(int64_t)token_req[t] * max_blocks + lp];
    if (page < 0) return;                                   // a table without a page here: checked on the host
    for (int i = threadIdx.x; i < K; i += kThreads) {
        const int g = i / dk, c = i - g * dk;
        kcache[((page * n_kv + g) * page_size + slot) * dk + c] =
            from_f32<T>(rot == 0 ? kp[i] * scale * k_gain[i] : turned(kp, k_gain, scale, i - c, c, rot, cs));
    }
    for (int i = threadIdx.x; i < V; i += kThreads) {
        const int g = i / dv, c = i - g * dv;
        vcache[((page * n_kv + g) * page_size + slot) * dv + c] = from_f32<T>(vp[i]);
    }
}

}  // namespace

// qkv float32 [n][H*dk + G*dk + G*dv] at row stride qkv_stride; q_out [n][H*dk] contiguous in the
// element type `dtype`, which is also the caches'.  kcache NULL: only q is produced (a layer
// that reads another layer's cache; qkv then holds the queries alone).  freq double [rot / 2], NULL with rot 0.
extern "C" int kllm_qknorm_append(void* q_out, const float* qkv, int64_t qkv_stride, const float* q_gain,
                                  const float* k_gain, float eps, float coef, int every, const int* positions,
                                  const int* token_req, const int* block_table, int max_blocks, void* kcache,
                                  void* vcache, int n, int n_heads, int n_kv, int dk, int dv, int page_size,
                                  int rot, const double* freq, int dtype, void* stream) {
    if (n <= 0) return 0;
    if (n_heads <= 0 || n_kv <= 0 || dk <= 0 || dv <= 0) KLLM_FAIL("qk norm: %d/%d heads of sizes %d/%d", n_heads, n_kv, dk, dv);
    if (coef != 0.f && every <= 0) KLLM_FAIL("qk norm: the temperature's period %d must be positive", every);
    if (rot < 0 || rot > dk || (rot & 1) || rot > kMaxRot || (rot > 0 && !freq))
        KLLM_FAIL("qk norm: rotary width %d invalid for head size %d", rot, dk);
    if (kcache && (page_size <= 0 || !vcache || !block_table)) KLLM_FAIL("qk norm: cache without pages or table");
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == KLLM_F32)
        kllm_launch((qknorm_append_kernel<float>), dim3(n), dim3(kThreads), 0, s, (float*)q_out, qkv, qkv_stride, q_gain,
                    k_gain, eps, coef, every, positions, token_req, block_table, max_blocks, (float*)kcache,
                    (float*)vcache, n_heads, n_kv, dk, dv, page_size, rot, freq);
    else if (dtype == KLLM_BF16)
        kllm_launch((qknorm_append_kernel<bf16>), dim3(n), dim3(kThreads), 0, s, (bf16*)q_out, qkv, qkv_stride, q_gain,
                    k_gain, eps, coef, every, positions, token_req, block_table, max_blocks, (bf16*)kcache,
                    (bf16*)vcache, n_heads, n_kv, dk, dv, page_size, rot, freq);
    else
        KLLM_FAIL("qk norm: unknown element type %d", dtype);
    KLLM_LAUNCH_STATUS();
}
