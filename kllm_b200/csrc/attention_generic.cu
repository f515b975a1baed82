// Causal grouped-query attention over the paged cache, generic form: any head
// size up to 512, values of their own size, any number of heads and kv heads, any query
// length, an optional window, an optional bias on the scores that is linear in the distance
// (slope[head] * (key position - query position)), an optional sink per head (a term of the
// softmax's denominator that has no key and no value), float32 arithmetic throughout.  It is the whole attention of
// the float32 path and the fallback of the bfloat16 path for head sizes that the
// tensor-core kernels do not take.
//
// One warp per (query token, head).  Keys are visited in chunks of 32 starting at
// the first visible key; lane i of the warp scores key i of the chunk, the running
// maximum and sum follow the online-softmax recurrence, and the lanes share the
// value accumulation by dimension.  A query at absolute position p sees keys
// [max(0, p + 1 - window), p]; the keys of its own step were appended before this
// kernel runs, so the loop bound is the whole mask (reference
// backend/model.cu:343-408: len = pos + 1, window start :361-362, scale after the
// dot :376, one division by the sum at the end :395-406).  The order of all sums
// depends on p and the window only, never on the batch or the cut of the prompt.
#include "common.cuh"

KLLM_EXPORT_LAST_ERROR(attention_generic)

namespace {

constexpr int kWarps = 4;
constexpr int kMaxHd = 512;

template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
attn_generic_kernel(T* __restrict__ out, const T* __restrict__ q, int64_t q_stride,
                    const T* __restrict__ kcache, const T* __restrict__ vcache,
                    const int* __restrict__ positions, const int* __restrict__ token_req,
                    const int* __restrict__ block_table, int max_blocks, int n_tokens,
                    int n_heads, int n_kv, int hd, int vd, int page_size, int window, float scale,
                    const float* __restrict__ slopes, const float* __restrict__ sinks, int segment, int v_heads,
                    int v_row, int out_f32) {
    __shared__ float qs[kWarps][kMaxHd];
    griddep_wait();
    griddep_launch();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t item = (int64_t)blockIdx.x * kWarps + warp;
    if (item >= (int64_t)n_tokens * n_heads) return;
    const int t = (int)(item / n_heads), h = (int)(item - (int64_t)t * n_heads);
    const int g = h / (n_heads / n_kv);
    const int p = positions[t];
    const int len = p + 1;
    int start = (window > 0 && len > window) ? len - window : 0;
    if (segment > 0) start = max(start, p - p % segment);          // a query sees only its own segment of positions
    const int gv = g / (n_kv / v_heads);                            // several key heads may share a value head
    const int* table = block_table + (int64_t)token_req[t] * max_blocks;

    const T* qr = q + (int64_t)t * q_stride + (int64_t)h * hd;
    for (int i = lane; i < hd; i += 32) qs[warp][i] = to_f32(qr[i]);
    __syncwarp();

    const float slope = slopes ? slopes[h] : 0.f;
    float acc[kMaxHd / 32];
#pragma unroll
    for (int i = 0; i < kMaxHd / 32; i++) acc[i] = 0.f;
    // a sink: one more term exp(sink[h]) in the softmax's denominator, without a key or a value
    float m = sinks ? sinks[h] : -INFINITY, l = sinks ? 1.f : 0.f;

    for (int base = start; base < len; base += 32) {
        const int key = base + lane;
        float sc = -INFINITY;
        int64_t row = 0;
        if (key < len) {
            const int page = table[key / page_size];
            row = ((int64_t)page * v_heads + gv) * page_size + (key % page_size);   // the key's row in the value store
            const T* kr = kcache + (((int64_t)page * n_kv + g) * page_size + (key % page_size)) * hd;
            float dot = 0.f;
            for (int d = 0; d < hd; d++) dot += qs[warp][d] * to_f32(kr[d]);
            sc = dot * scale + slope * (float)(key - p);
        }
        const float m_new = fmaxf(m, warp_max(sc));
        const float corr = expf(m - m_new);  // 0 on the first chunk (m = -inf)
        const float pr = (key < len) ? expf(sc - m_new) : 0.f;
        l = l * corr + warp_sum(pr);
        m = m_new;
#pragma unroll
        for (int i = 0; i < kMaxHd / 32; i++) acc[i] *= corr;
        const int cnt = min(32, len - base);
        for (int j = 0; j < cnt; j++) {
            const float pj = __shfl_sync(0xffffffffu, pr, j);
            const int64_t rj = __shfl_sync(0xffffffffu, row, j);
            const T* vr = vcache + rj * v_row;
#pragma unroll
            for (int i = 0; i < kMaxHd / 32; i++) {
                const int d = lane + 32 * i;
                if (d < vd) acc[i] += pj * to_f32(vr[d]);
            }
        }
    }
    const float inv = 1.f / l;
    const int64_t o0 = (int64_t)t * n_heads * vd + (int64_t)h * vd;
#pragma unroll
    for (int i = 0; i < kMaxHd / 32; i++) {
        const int d = lane + 32 * i;
        if (d < vd) {
            if (out_f32) reinterpret_cast<float*>(out)[o0 + d] = acc[i] * inv;
            else out[o0 + d] = from_f32<T>(acc[i] * inv);
        }
    }
}

}  // namespace

// out [n, n_heads*vd]; q rows of n_heads*hd at stride q_stride (elements);
// caches [pages, n_kv, page_size, hd] and [pages, n_kv, page_size, vd]; block_table
// [requests, max_blocks]; slopes optional float32 [n_heads]; sinks optional float32 [n_heads]:
// exp(sinks[h]) is added to the denominator of head h's softmax (unscaled, once).
// segment > 0: a query sees only the keys of its own segment of that many positions (counted from 0);
// v_heads: heads of the value store (n_kv / v_heads neighbouring key heads read one value head);
// v_row: elements between two value rows; out_f32: `out` is float32 whatever the operands' type.
extern "C" int kllm_attention_generic(void* out, const void* q, int64_t q_stride,
                                      const void* kcache, const void* vcache,
                                      const int* positions, const int* token_req,
                                      const int* block_table, int max_blocks, int n_tokens,
                                      int n_heads, int n_kv, int hd, int vd, int page_size, int window,
                                      float scale, const float* slopes, const float* sinks, int segment,
                                      int v_heads, int v_row, int out_f32, int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    if (hd <= 0 || hd > kMaxHd) KLLM_FAIL("attention: head size %d not in 1..%d", hd, kMaxHd);
    if (vd <= 0 || vd > kMaxHd) KLLM_FAIL("attention: value size %d not in 1..%d", vd, kMaxHd);
    if (n_kv <= 0 || n_heads % n_kv) KLLM_FAIL("attention: %d heads over %d kv heads", n_heads, n_kv);
    if (page_size <= 0) KLLM_FAIL("attention: page size %d", page_size);
    if (segment < 0 || v_heads <= 0 || n_kv % v_heads || v_row < vd)
        KLLM_FAIL("attention: segment %d, %d value heads under %d key heads, value rows of %d at a stride of %d", segment,
                  v_heads, n_kv, vd, v_row);
    cudaStream_t s = (cudaStream_t)stream;
    const int64_t items = (int64_t)n_tokens * n_heads;
    const unsigned grid = (unsigned)((items + kWarps - 1) / kWarps);
    if (dtype == KLLM_F32)
        kllm_launch((attn_generic_kernel<float>), dim3(grid), dim3(kWarps * 32), 0, s, 
            (float*)out, (const float*)q, q_stride, (const float*)kcache, (const float*)vcache,
            positions, token_req, block_table, max_blocks, n_tokens, n_heads, n_kv, hd, vd, page_size,
            window, scale, slopes, sinks, segment, v_heads, v_row, out_f32);
    else if (dtype == KLLM_BF16)
        kllm_launch((attn_generic_kernel<bf16>), dim3(grid), dim3(kWarps * 32), 0, s, 
            (bf16*)out, (const bf16*)q, q_stride, (const bf16*)kcache, (const bf16*)vcache,
            positions, token_req, block_table, max_blocks, n_tokens, n_heads, n_kv, hd, vd, page_size,
            window, scale, slopes, sinks, segment, v_heads, v_row, out_f32);
    else
        KLLM_FAIL("attention: unknown element type %d", dtype);
    KLLM_LAUNCH_STATUS();
}
