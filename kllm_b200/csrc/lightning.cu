// Linear attention with one fixed decay per head ("lightning attention"), for mixed batches of
// prompt portions and single tokens, with the state of every request in a slot of a state tensor.
//
// Per head, with dk key channels, dv value channels, a decay w in (0, 1] and a state S [dk][dv]
// that starts at zero for a new request:
//
//     q, k, v = silu of the head's parts of the projections
//     S_t = w S_(t-1) + k_t v_t^T            o_t = S_t^T q_t
//
// Everything is float32: the projections arrive unrounded, the activation, the powers of the
// decay, the state and the sums.  A request's rows are taken in chunks of up to C rows; inside a
// chunk that starts with the state S,
//
//     o_i = w^(i+1) S^T q_i + sum over j <= i of w^(i-j) (q_i . k_j) v_j
//     S'  = w^n S + sum over j of w^(n-1-j) k_j v_j^T                          (n rows in the chunk)
//
// which is the recurrence written out, so a prompt cut anywhere gives the same sums up to their
// order.  A CTA takes (head, slice of value channels, request): it keeps its [dk][slice] part of
// the state in shared memory from the first chunk to the last and writes it back to the slot.
// A single decoded token is a chunk of one row.  Steps that hold portions take two kernels instead (further down):
// the chunks' own sums, which need no state, for all chunks at once, then the state's walk over the chunks.
//
// The second kernel joins the heads: y = o / rms(o over ALL heads' values) * gain * sigmoid(g).
#include "common.cuh"

KLLM_EXPORT_LAST_ERROR(lightning)

namespace {

constexpr int kChunk = 32;
constexpr int kThreads = 256;

__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }

// grid (heads * slices, requests).  Shared memory: S [dk][sl], q [C][dk + 1], k [C][dk + 1], v [C][sl],
// A [C][C + 1], pw [C + 1].
__global__ void __launch_bounds__(kThreads)
lightning_scan_kernel(float* __restrict__ o, int64_t o_stride, const float* __restrict__ q, int64_t q_stride,
                      const float* __restrict__ k, int64_t k_stride, const float* __restrict__ v, int64_t v_stride,
                      const float* __restrict__ decay, float* __restrict__ state, int64_t state_stride,
                      const int* __restrict__ q_start, const int* __restrict__ state_slots, int heads, int dk, int dv,
                      int sl, int slices) {
    extern __shared__ float sm[];
    const int head = blockIdx.x / slices, slice = blockIdx.x - head * slices;
    const int e0 = slice * sl, ne = min(sl, dv - e0);
    const int req = blockIdx.y;
    const int qp = dk + 1;
    float* S = sm;                          // [dk][sl]
    float* qs = S + dk * sl;                // [C][dk + 1]
    float* ks = qs + kChunk * qp;           // [C][dk + 1]
    float* vs = ks + kChunk * qp;           // [C][sl]
    float* A = vs + kChunk * sl;            // [C][C + 1]
    float* pw = A + kChunk * (kChunk + 1);  // [C + 1]: w^0 .. w^C
    const int tid = threadIdx.x;
    const float w = decay[head];
    if (tid <= kChunk) pw[tid] = (float)pow((double)w, (double)tid);
    griddep_wait();
    griddep_launch();
    const int row0 = q_start[req], row1 = q_start[req + 1];
    float* slot = state + (int64_t)state_slots[req] * state_stride + (int64_t)head * dk * dv;
    for (int i = tid; i < dk * ne; i += kThreads) {
        const int d = i / ne, e = i - d * ne;
        S[d * sl + e] = slot[(int64_t)d * dv + e0 + e];
    }
    for (int c0 = row0; c0 < row1; c0 += kChunk) {
        const int n = min(kChunk, row1 - c0);
        __syncthreads();                    // the chunk before has been used up; S and pw are written
        for (int i = tid; i < n * dk; i += kThreads) {
            const int r = i / dk, d = i - r * dk;
            qs[r * qp + d] = silu_f(q[(int64_t)(c0 + r) * q_stride + head * dk + d]);
            ks[r * qp + d] = silu_f(k[(int64_t)(c0 + r) * k_stride + head * dk + d]);
        }
        for (int i = tid; i < n * ne; i += kThreads) {
            const int r = i / ne, e = i - r * ne;
            vs[r * sl + e] = silu_f(v[(int64_t)(c0 + r) * v_stride + head * dv + e0 + e]);
        }
        __syncthreads();
        // A[i][j] = w^(i-j) q_i . k_j for j <= i
        for (int it = tid; it < n * n; it += kThreads) {
            const int i = it / n, j = it - i * n;
            float a = 0.f;
            if (j <= i) {
                const float* qi = qs + i * qp;
                const float* kj = ks + j * qp;
                float b = 0.f;
                int d = 0;
                for (; d + 1 < dk; d += 2) {
                    a = fmaf(qi[d], kj[d], a);
                    b = fmaf(qi[d + 1], kj[d + 1], b);
                }
                if (d < dk) a = fmaf(qi[d], kj[d], a);
                a = (a + b) * pw[i - j];
            }
            A[i * (kChunk + 1) + j] = a;
        }
        __syncthreads();
        // o_i[e] = w^(i+1) sum_d S[d][e] q_i[d] + sum_{j<=i} A[i][j] v_j[e]: a thread takes four rows i of one channel e,
        // so that a value of S or v read from shared memory serves four sums (A is zero above its diagonal)
        const int ib = (n + 3) / 4;
        for (int it = tid; it < ib * ne; it += kThreads) {
            const int i0 = (it / ne) * 4, e = it - (it / ne) * ne;
            const float* q0 = qs + i0 * qp;
            const float* q1 = qs + min(i0 + 1, n - 1) * qp;
            const float* q2 = qs + min(i0 + 2, n - 1) * qp;
            const float* q3 = qs + min(i0 + 3, n - 1) * qp;
            float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll 4
            for (int d = 0; d < dk; d++) {
                const float sv = S[d * sl + e];
                a0 = fmaf(sv, q0[d], a0);
                a1 = fmaf(sv, q1[d], a1);
                a2 = fmaf(sv, q2[d], a2);
                a3 = fmaf(sv, q3[d], a3);
            }
            a0 *= pw[i0 + 1];
            a1 *= pw[min(i0 + 2, kChunk)];
            a2 *= pw[min(i0 + 3, kChunk)];
            a3 *= pw[min(i0 + 4, kChunk)];
            const float* A0 = A + i0 * (kChunk + 1);
            const float* A1 = A + min(i0 + 1, n - 1) * (kChunk + 1);
            const float* A2 = A + min(i0 + 2, n - 1) * (kChunk + 1);
            const float* A3 = A + min(i0 + 3, n - 1) * (kChunk + 1);
            const int jn = min(n, i0 + 4);
#pragma unroll 4
            for (int j = 0; j < jn; j++) {
                const float vv = vs[j * sl + e];
                a0 = fmaf(A0[j], vv, a0);
                a1 = fmaf(A1[j], vv, a1);
                a2 = fmaf(A2[j], vv, a2);
                a3 = fmaf(A3[j], vv, a3);
            }
            float* orow = o + (int64_t)(c0 + i0) * o_stride + head * dv + e0 + e;
            orow[0] = a0;
            if (i0 + 1 < n) orow[o_stride] = a1;
            if (i0 + 2 < n) orow[2 * o_stride] = a2;
            if (i0 + 3 < n) orow[3 * o_stride] = a3;
        }
        __syncthreads();
        // S[d][e] = w^n S[d][e] + sum_j w^(n-1-j) k_j[d] v_j[e]: a thread takes four key channels d of one channel e
        const int db = (dk + 3) / 4;
        for (int it = tid; it < db * ne; it += kThreads) {
            const int d0 = (it / ne) * 4, e = it - (it / ne) * ne;
            const int d1 = min(d0 + 1, dk - 1), d2 = min(d0 + 2, dk - 1), d3 = min(d0 + 3, dk - 1);
            float a0 = S[d0 * sl + e] * pw[n], a1 = S[d1 * sl + e] * pw[n], a2 = S[d2 * sl + e] * pw[n], a3 = S[d3 * sl + e] * pw[n];
#pragma unroll 4
            for (int j = 0; j < n; j++) {
                const float vv = vs[j * sl + e] * pw[n - 1 - j];
                const float* kj = ks + j * qp;
                a0 = fmaf(kj[d0], vv, a0);
                a1 = fmaf(kj[d1], vv, a1);
                a2 = fmaf(kj[d2], vv, a2);
                a3 = fmaf(kj[d3], vv, a3);
            }
            S[d0 * sl + e] = a0;
            if (d0 + 1 < dk) S[(d0 + 1) * sl + e] = a1;
            if (d0 + 2 < dk) S[(d0 + 2) * sl + e] = a2;
            if (d0 + 3 < dk) S[(d0 + 3) * sl + e] = a3;
        }
    }
    __syncthreads();
    for (int i = tid; i < dk * ne; i += kThreads) {
        const int d = i / ne, e = i - d * ne;
        slot[(int64_t)d * dv + e0 + e] = S[d * sl + e];
    }
}

// ---- portions: the chunk's own part in parallel, the state's part in sequence ----------------------------------
// The sum inside a chunk, sum over j <= i of w^(i-j) (q_i . k_j) v_j, needs nothing of the state: one CTA per
// (chunk, head) forms it for all chunks of the step at once, and leaves silu(q), silu(k), silu(v) in float32 work
// rows for the second kernel, which walks a request's chunks in order with its slice of the state in shared memory and
// adds w^(i+1) S^T q_i to the rows before it moves S on.  Both cut a request's rows of the step into the same chunks.
constexpr int kPitchPad = 4;    // rows of q and k in shared memory start on 16-byte boundaries (float4 reads)

// grid (chunk bound, heads).  Shared memory: q [C][dk + 1], k [C][dk + 1], v [C][dv], A [C][C + 1], pw [C + 1].
__global__ void __launch_bounds__(kThreads)
lightning_chunk_kernel(float* __restrict__ o, int64_t o_stride, float* __restrict__ qa, float* __restrict__ ka,
                       float* __restrict__ va, const float* __restrict__ q, int64_t q_stride, const float* __restrict__ k,
                       int64_t k_stride, const float* __restrict__ v, int64_t v_stride, const float* __restrict__ decay,
                       const int* __restrict__ q_start, int n_requests, int heads, int dk, int dv) {
    extern __shared__ float sm[];
    const int head = blockIdx.y;
    const int qp = dk + 1;
    float* qs = sm;
    float* ks = qs + kChunk * qp;
    float* vs = ks + kChunk * qp;                   // [C][dv]
    float* A = vs + kChunk * dv;
    float* pw = A + kChunk * (kChunk + 1);
    const int tid = threadIdx.x;
    if (tid <= kChunk) pw[tid] = (float)pow((double)decay[head], (double)tid);
    griddep_wait();
    griddep_launch();
    int req = 0, chunk = blockIdx.x;
    for (; req < n_requests; req++) {
        const int chunks = (q_start[req + 1] - q_start[req] + kChunk - 1) / kChunk;
        if (chunk < chunks) break;
        chunk -= chunks;
    }
    if (req >= n_requests) return;
    const int c0 = q_start[req] + chunk * kChunk;
    const int n = min(kChunk, q_start[req + 1] - c0);
    const int A_w = heads * dk, B_w = heads * dv;
    for (int i = tid; i < n * dk; i += kThreads) {
        const int r = i / dk, d = i - r * dk;
        const float qv = silu_f(q[(int64_t)(c0 + r) * q_stride + head * dk + d]);
        const float kv = silu_f(k[(int64_t)(c0 + r) * k_stride + head * dk + d]);
        qs[r * qp + d] = qv;
        ks[r * qp + d] = kv;
        qa[(int64_t)(c0 + r) * A_w + head * dk + d] = qv;
        ka[(int64_t)(c0 + r) * A_w + head * dk + d] = kv;
    }
    for (int i = tid; i < n * dv; i += kThreads) {
        const int r = i / dv, e = i - r * dv;
        const float vv = silu_f(v[(int64_t)(c0 + r) * v_stride + head * dv + e]);
        vs[r * dv + e] = vv;
        va[(int64_t)(c0 + r) * B_w + head * dv + e] = vv;
    }
    __syncthreads();
    for (int it = tid; it < n * n; it += kThreads) {
        const int i = it / n, j = it - i * n;
        float a = 0.f;
        if (j <= i) {
            const float* qi = qs + i * qp;
            const float* kj = ks + j * qp;
            float b = 0.f;
            int d = 0;
            for (; d + 1 < dk; d += 2) {
                a = fmaf(qi[d], kj[d], a);
                b = fmaf(qi[d + 1], kj[d + 1], b);
            }
            if (d < dk) a = fmaf(qi[d], kj[d], a);
            a = (a + b) * pw[i - j];
        }
        A[i * (kChunk + 1) + j] = a;
    }
    __syncthreads();
    const int ib = (n + 3) / 4;
    for (int it = tid; it < ib * dv; it += kThreads) {
        const int i0 = (it / dv) * 4, e = it - (it / dv) * dv;
        const float* A0 = A + i0 * (kChunk + 1);
        const float* A1 = A + min(i0 + 1, n - 1) * (kChunk + 1);
        const float* A2 = A + min(i0 + 2, n - 1) * (kChunk + 1);
        const float* A3 = A + min(i0 + 3, n - 1) * (kChunk + 1);
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
        const int jn = min(n, i0 + 4);
#pragma unroll 4
        for (int j = 0; j < jn; j++) {
            const float vv = vs[j * dv + e];
            a0 = fmaf(A0[j], vv, a0);
            a1 = fmaf(A1[j], vv, a1);
            a2 = fmaf(A2[j], vv, a2);
            a3 = fmaf(A3[j], vv, a3);
        }
        float* orow = o + (int64_t)(c0 + i0) * o_stride + head * dv + e;
        orow[0] = a0;
        if (i0 + 1 < n) orow[o_stride] = a1;
        if (i0 + 2 < n) orow[2 * o_stride] = a2;
        if (i0 + 3 < n) orow[3 * o_stride] = a3;
    }
}

// grid (heads * slices, requests).  Shared memory: S [dk][sl], q [C][dk + 4], k [C][dk + 4], v [C][sl], pw [C + 1];
// dk a multiple of 4.  o already holds the chunks' own sums.
__global__ void __launch_bounds__(kThreads)
lightning_state_kernel(float* __restrict__ o, int64_t o_stride, const float* __restrict__ qa, const float* __restrict__ ka,
                       const float* __restrict__ va, const float* __restrict__ decay, float* __restrict__ state,
                       int64_t state_stride, const int* __restrict__ q_start, const int* __restrict__ state_slots,
                       int heads, int dk, int dv, int sl, int slices) {
    extern __shared__ __align__(16) float sm[];
    const int head = blockIdx.x / slices, slice = blockIdx.x - head * slices;
    const int e0 = slice * sl, ne = min(sl, dv - e0);
    const int req = blockIdx.y;
    const int qp = dk + kPitchPad;
    float* S = sm;                          // [dk][sl]
    float* qs = S + dk * sl;                // [C][qp]
    float* ks = qs + kChunk * qp;
    float* vs = ks + kChunk * qp;           // [C][sl]
    float* pw = vs + kChunk * sl;
    const int tid = threadIdx.x;
    if (tid <= kChunk) pw[tid] = (float)pow((double)decay[head], (double)tid);
    griddep_wait();
    griddep_launch();
    const int row0 = q_start[req], row1 = q_start[req + 1];
    const int A_w = heads * dk, B_w = heads * dv;
    float* slot = state + (int64_t)state_slots[req] * state_stride + (int64_t)head * dk * dv;
    for (int i = tid; i < dk * ne; i += kThreads) {
        const int d = i / ne, e = i - d * ne;
        S[d * sl + e] = slot[(int64_t)d * dv + e0 + e];
    }
    const int dk4 = dk / 4;
    for (int c0 = row0; c0 < row1; c0 += kChunk) {
        const int n = min(kChunk, row1 - c0);
        __syncthreads();
        for (int i = tid; i < n * dk4; i += kThreads) {
            const int r = i / dk4, d = (i - r * dk4) * 4;
            *reinterpret_cast<float4*>(qs + r * qp + d) = *reinterpret_cast<const float4*>(qa + (int64_t)(c0 + r) * A_w + head * dk + d);
            *reinterpret_cast<float4*>(ks + r * qp + d) = *reinterpret_cast<const float4*>(ka + (int64_t)(c0 + r) * A_w + head * dk + d);
        }
        for (int i = tid; i < n * ne; i += kThreads) {
            const int r = i / ne, e = i - r * ne;
            vs[r * sl + e] = va[(int64_t)(c0 + r) * B_w + head * dv + e0 + e];
        }
        __syncthreads();
        // o_i[e] += w^(i+1) sum_d S[d][e] q_i[d]: four rows a thread, four key channels a step
        const int ib = (n + 3) / 4;
        for (int it = tid; it < ib * ne; it += kThreads) {
            const int i0 = (it / ne) * 4, e = it - (it / ne) * ne;
            const float* q0 = qs + i0 * qp;
            const float* q1 = qs + min(i0 + 1, n - 1) * qp;
            const float* q2 = qs + min(i0 + 2, n - 1) * qp;
            const float* q3 = qs + min(i0 + 3, n - 1) * qp;
            float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
            for (int d = 0; d < dk; d += 4) {
                const float s0 = S[d * sl + e], s1 = S[(d + 1) * sl + e], s2 = S[(d + 2) * sl + e], s3 = S[(d + 3) * sl + e];
                const float4 x0 = *reinterpret_cast<const float4*>(q0 + d), x1 = *reinterpret_cast<const float4*>(q1 + d);
                const float4 x2 = *reinterpret_cast<const float4*>(q2 + d), x3 = *reinterpret_cast<const float4*>(q3 + d);
                a0 = fmaf(s0, x0.x, a0); a0 = fmaf(s1, x0.y, a0); a0 = fmaf(s2, x0.z, a0); a0 = fmaf(s3, x0.w, a0);
                a1 = fmaf(s0, x1.x, a1); a1 = fmaf(s1, x1.y, a1); a1 = fmaf(s2, x1.z, a1); a1 = fmaf(s3, x1.w, a1);
                a2 = fmaf(s0, x2.x, a2); a2 = fmaf(s1, x2.y, a2); a2 = fmaf(s2, x2.z, a2); a2 = fmaf(s3, x2.w, a2);
                a3 = fmaf(s0, x3.x, a3); a3 = fmaf(s1, x3.y, a3); a3 = fmaf(s2, x3.z, a3); a3 = fmaf(s3, x3.w, a3);
            }
            float* orow = o + (int64_t)(c0 + i0) * o_stride + head * dv + e0 + e;
            orow[0] += a0 * pw[i0 + 1];
            if (i0 + 1 < n) orow[o_stride] += a1 * pw[i0 + 2];
            if (i0 + 2 < n) orow[2 * o_stride] += a2 * pw[i0 + 3];
            if (i0 + 3 < n) orow[3 * o_stride] += a3 * pw[i0 + 4];
        }
        __syncthreads();
        // S[d][e] = w^n S[d][e] + sum_j w^(n-1-j) k_j[d] v_j[e]: four key channels a thread
        for (int it = tid; it < dk4 * ne; it += kThreads) {
            const int d0 = (it / ne) * 4, e = it - (it / ne) * ne;
            float a0 = S[d0 * sl + e] * pw[n], a1 = S[(d0 + 1) * sl + e] * pw[n], a2 = S[(d0 + 2) * sl + e] * pw[n],
                  a3 = S[(d0 + 3) * sl + e] * pw[n];
#pragma unroll 4
            for (int j = 0; j < n; j++) {
                const float vv = vs[j * sl + e] * pw[n - 1 - j];
                const float4 kk = *reinterpret_cast<const float4*>(ks + j * qp + d0);
                a0 = fmaf(kk.x, vv, a0);
                a1 = fmaf(kk.y, vv, a1);
                a2 = fmaf(kk.z, vv, a2);
                a3 = fmaf(kk.w, vv, a3);
            }
            S[d0 * sl + e] = a0;
            S[(d0 + 1) * sl + e] = a1;
            S[(d0 + 2) * sl + e] = a2;
            S[(d0 + 3) * sl + e] = a3;
        }
    }
    __syncthreads();
    for (int i = tid; i < dk * ne; i += kThreads) {
        const int d = i / ne, e = i - d * ne;
        slot[(int64_t)d * dv + e0 + e] = S[d * sl + e];
    }
}

size_t chunk_smem(int dk, int dv) {
    return sizeof(float) * (2 * (size_t)kChunk * (dk + 1) + (size_t)kChunk * dv + (size_t)kChunk * (kChunk + 1) + kChunk + 1);
}

size_t state_smem(int dk, int sl) {
    return sizeof(float) * ((size_t)dk * sl + 2 * (size_t)kChunk * (dk + kPitchPad) + (size_t)kChunk * sl + kChunk + 4);
}

// y[t,:] = o[t,:] * rsqrt(mean over all `width` values of o[t,:]^2 + eps) * gain * sigmoid(g[t,:]); one CTA per row.
template <typename T>
__global__ void __launch_bounds__(kThreads)
gate_norm_kernel(T* __restrict__ y, const float* __restrict__ o, int64_t o_stride, const float* __restrict__ g,
                 int64_t g_stride, const float* __restrict__ gain, int width, float eps) {
    __shared__ float red[32];
    griddep_wait();
    griddep_launch();
    const int t = blockIdx.x;
    const float* orow = o + (int64_t)t * o_stride;
    const float* grow = g + (int64_t)t * g_stride;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += kThreads) ss += orow[i] * orow[i];
    ss = block_sum(ss, red);
    const float scale = rsqrtf(ss / (float)width + eps);
    T* yr = y + (int64_t)t * width;
    for (int i = threadIdx.x; i < width; i += kThreads)
        yr[i] = from_f32<T>(orow[i] * scale * gain[i] / (1.f + expf(-grow[i])));
}

size_t scan_smem(int dk, int sl) {
    return sizeof(float) * ((size_t)dk * sl + 2 * (size_t)kChunk * (dk + 1) + (size_t)kChunk * sl +
                            (size_t)kChunk * (kChunk + 1) + kChunk + 1);
}

}  // namespace

// o float32 [n][heads * dv]; q, k float32 rows of heads * dk, v float32 rows of heads * dv (the projections,
// before their activation), each at its row stride; decay float32 [heads]; state float32 [slots][state_stride]
// whose first heads * dk * dv values are S as [heads][dk][dv]; q_start int32 [requests + 1], state_slots int32
// [requests].
extern "C" int kllm_lightning_scan(float* o, int64_t o_stride, const float* q, int64_t q_stride, const float* k,
                                   int64_t k_stride, const float* v, int64_t v_stride, const float* decay, float* state,
                                   int64_t state_stride, const int* q_start, const int* state_slots, int n,
                                   int n_requests, int heads, int dk, int dv, void* stream) {
    if (n <= 0 || n_requests <= 0) return 0;
    if (heads <= 0 || dk <= 0 || dv <= 0) KLLM_FAIL("lightning scan: %d heads of sizes %d, %d", heads, dk, dv);
    if (n_requests > 65535) KLLM_FAIL("lightning scan: %d requests in one launch", n_requests);
    if (state_stride < (int64_t)heads * dk * dv) KLLM_FAIL("lightning scan: a state slot of %lld values is too small", (long long)state_stride);
    // the slice of value channels: as wide as the shared memory of a CTA holds beside the chunk, at most 64
    int sl = dv < 64 ? dv : 64;
    while (sl > 1 && scan_smem(dk, sl) > 200 * 1024) sl = (sl + 1) / 2;
    if (scan_smem(dk, sl) > 200 * 1024) KLLM_FAIL("lightning scan: a head of %d key channels does not fit shared memory", dk);
    // a launch of few (head, request) pairs gets narrower slices, down to 16 channels: more CTAs, each repeating the
    // chunk's small q k^T product
    while (sl > 16 && (int64_t)heads * n_requests * ((dv + sl - 1) / sl) < 148) sl = (sl + 1) / 2;
    const int slices = (dv + sl - 1) / sl;
    const size_t smem = scan_smem(dk, sl);
    static size_t allowed = 48 * 1024;
    if (smem > allowed) {
        cudaError_t e = cudaFuncSetAttribute(lightning_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) KLLM_FAIL("lightning scan: %s", cudaGetErrorString(e));
        allowed = 200 * 1024;
    }
    kllm_launch((lightning_scan_kernel), dim3(heads * slices, n_requests), dim3(kThreads), smem, (cudaStream_t)stream, o,
                o_stride, q, q_stride, k, k_stride, v, v_stride, decay, state, state_stride, q_start, state_slots, heads,
                dk, dv, sl, slices);
    KLLM_LAUNCH_STATUS();
}

// y [n][width] contiguous in the element type `dtype`; o, g float32 rows of `width` values at their strides;
// gain float32 [width].
extern "C" int kllm_lightning_gate_norm(void* y, const float* o, int64_t o_stride, const float* g, int64_t g_stride,
                                        const float* gain, int n, int width, float eps, int dtype, void* stream) {
    if (n <= 0) return 0;
    if (width <= 0) KLLM_FAIL("lightning gate norm: width %d", width);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == KLLM_F32)
        kllm_launch((gate_norm_kernel<float>), dim3(n), dim3(kThreads), 0, s, (float*)y, o, o_stride, g, g_stride, gain,
                    width, eps);
    else if (dtype == KLLM_BF16)
        kllm_launch((gate_norm_kernel<bf16>), dim3(n), dim3(kThreads), 0, s, (bf16*)y, o, o_stride, g, g_stride, gain,
                    width, eps);
    else
        KLLM_FAIL("lightning gate norm: unknown element type %d", dtype);
    KLLM_LAUNCH_STATUS();
}

// The same recurrence for steps that hold portions, in two kernels (see above): work float32 [3][n][heads * max(dk, dv)]
// rows for silu(q), silu(k), silu(v); chunk_bound: an upper bound of the chunks (sum over requests of ceil(rows / 32)).
// Returns -3 when the sizes are not taken (dk no multiple of 4, or shared memory), for the caller to use kllm_lightning_scan.
extern "C" int kllm_lightning_scan_portions(float* o, int64_t o_stride, const float* q, int64_t q_stride, const float* k,
                                            int64_t k_stride, const float* v, int64_t v_stride, const float* decay,
                                            float* state, int64_t state_stride, const int* q_start, const int* state_slots,
                                            int n, int n_requests, int chunk_bound, int heads, int dk, int dv, float* qa,
                                            float* ka, float* va, void* stream) {
    if (n <= 0 || n_requests <= 0) return 0;
    if (heads <= 0 || dk <= 0 || dv <= 0) KLLM_FAIL("lightning scan: %d heads of sizes %d, %d", heads, dk, dv);
    if (n_requests > 65535 || heads > 65535) KLLM_FAIL("lightning scan: %d requests, %d heads in one launch", n_requests, heads);
    if (state_stride < (int64_t)heads * dk * dv) KLLM_FAIL("lightning scan: a state slot of %lld values is too small", (long long)state_stride);
    if (dk % 4 || (heads * dk) % 4 || (((uintptr_t)qa | (uintptr_t)ka) & 15) || chunk_smem(dk, dv) > 200 * 1024) return -3;
    int sl = dv < 32 ? dv : 32;
    while (sl > 1 && state_smem(dk, sl) > 200 * 1024) sl = (sl + 1) / 2;
    if (state_smem(dk, sl) > 200 * 1024) return -3;
    while (sl > 16 && (int64_t)heads * n_requests * ((dv + sl - 1) / sl) < 148) sl = (sl + 1) / 2;
    const int slices = (dv + sl - 1) / sl;
    static bool raised = false;
    if (!raised) {
        cudaFuncSetAttribute(lightning_chunk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        cudaFuncSetAttribute(lightning_state_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        raised = true;
    }
    cudaStream_t s = (cudaStream_t)stream;
    kllm_launch((lightning_chunk_kernel), dim3(chunk_bound, heads), dim3(kThreads), chunk_smem(dk, dv), s, o, o_stride, qa, ka, va,
                q, q_stride, k, k_stride, v, v_stride, decay, q_start, n_requests, heads, dk, dv);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) KLLM_FAIL("lightning scan: %s", cudaGetErrorString(e));
    kllm_launch((lightning_state_kernel), dim3(heads * slices, n_requests), dim3(kThreads), state_smem(dk, sl), s, o, o_stride, qa, ka,
                va, decay, state, state_stride, q_start, state_slots, heads, dk, dv, sl, slices);
    KLLM_LAUNCH_STATUS();
}
