// RMSNorm with the residual sum folded in.
//
//   x[r,:] (+)= res[r,:]          residual stream, float32, written back
//   out[r,:] = x[r,:] * rsqrt(mean(x^2) + eps) * gain[:]
//
// The sum of squares, the scale and the residual sum are float32 whatever the
// element types of `res` and `out` are (res may be float32 beside a bfloat16 out:
// a projection's float32 result goes into the residual stream unrounded).  One block per row; the order of the
// additions depends on the row width and the block size only.
// Formula: reference backend/model.cu:101-122 (norm) and :144-165 (sum + norm).
#include "common.cuh"

KLLM_EXPORT_LAST_ERROR(norm)

namespace {

constexpr int kThreads = 256;

// rows == nullptr: row r of x/res, x is written back.
// rows != nullptr: row rows[r] of x/res is read, nothing is written back (used to
// normalise only the rows whose logits are wanted).
template <typename T, typename R>
__global__ void __launch_bounds__(kThreads)
add_rmsnorm_kernel(float* __restrict__ x, const R* __restrict__ res, T* __restrict__ out,
                   const float* __restrict__ gain, const int* __restrict__ rows,
                   int d, float eps) {
    __shared__ float red[32];
    griddep_wait();
    griddep_launch();
    const int r = blockIdx.x;
    const int64_t src = rows ? (int64_t)rows[r] : (int64_t)r;
    float* xr = x + src * d;
    const R* rr = res ? res + src * d : nullptr;
    T* orow = out + (int64_t)r * d;
    const bool write_back = (rows == nullptr) && (res != nullptr);

    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += kThreads) {
        float v = xr[i];
        if (rr) {
            v += to_f32(rr[i]);
            if (write_back) xr[i] = v;
        }
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float scale = rsqrtf(ss / (float)d + eps);
    for (int i = threadIdx.x; i < d; i += kThreads) {
        float v = xr[i];
        if (rr && !write_back) v += to_f32(rr[i]);
        orow[i] = from_f32<T>(v * scale * gain[i]);
    }
}

// The common case of a step's rows (every row, float32 residual or none, bfloat16 out,
// width a multiple of 4 up to kThreads * 4 * kVec) in one pass: a thread keeps its
// elements in registers between the sum of squares and the scaling, 16-byte accesses.
// Same sums in the same order as the kernel above: thread k adds its elements i = k,
// k + kThreads, ... in that order (here four neighbours at a time, whose squares are
// added first; a rounding may differ from the scalar kernel's).
constexpr int kVec = 8;

__global__ void __launch_bounds__(kThreads)
add_rmsnorm_vec4_kernel(float* __restrict__ x, const float* __restrict__ res, bf16* __restrict__ out,
                        const float* __restrict__ gain, int d, float eps) {
    __shared__ float red[32];
    griddep_wait();
    griddep_launch();
    const int r = blockIdx.x;
    float4* xr = reinterpret_cast<float4*>(x + (int64_t)r * d);
    const float4* rr = res ? reinterpret_cast<const float4*>(res + (int64_t)r * d) : nullptr;
    const float4* g4 = reinterpret_cast<const float4*>(gain);
    const int n4 = d >> 2;
    float4 v[kVec];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < kVec; k++) {
        const int i = threadIdx.x + k * kThreads;
        if (i < n4) {
            v[k] = xr[i];
            if (rr) {
                const float4 a = rr[i];
                v[k].x += a.x; v[k].y += a.y; v[k].z += a.z; v[k].w += a.w;
                xr[i] = v[k];
            }
            ss += (v[k].x * v[k].x + v[k].y * v[k].y) + (v[k].z * v[k].z + v[k].w * v[k].w);
        }
    }
    ss = block_sum(ss, red);
    const float scale = rsqrtf(ss / (float)d + eps);
    uint2* orow = reinterpret_cast<uint2*>(out + (int64_t)r * d);
#pragma unroll
    for (int k = 0; k < kVec; k++) {
        const int i = threadIdx.x + k * kThreads;
        if (i < n4) {
            const float4 g = g4[i];
            __nv_bfloat162 lo = __floats2bfloat162_rn(v[k].x * scale * g.x, v[k].y * scale * g.y);
            __nv_bfloat162 hi = __floats2bfloat162_rn(v[k].z * scale * g.z, v[k].w * scale * g.w);
            uint2 pk;
            pk.x = *reinterpret_cast<uint32_t*>(&lo);
            pk.y = *reinterpret_cast<uint32_t*>(&hi);
            orow[i] = pk;
        }
    }
}

// One warp per row, the row in registers, no block-wide synchronisation; 8 rows per CTA.
// Width a multiple of 4 up to 32 * 4 * kWarpVec.  Lane l adds the squares of its float4 l,
// l + 32, ... in that order, then the lanes are added in a fixed tree.  Which of the two
// vectorised kernels runs is decided by the width alone, never by the number of rows, so
// a row is summed in the same order whatever else the step holds.
constexpr int kWarpVec = 16;

__global__ void __launch_bounds__(256)
add_rmsnorm_warp_kernel(float* __restrict__ x, const float* __restrict__ res, bf16* __restrict__ out,
                        const float* __restrict__ gain, int n_rows, int d, float eps) {
    griddep_wait();
    griddep_launch();
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (r >= n_rows) return;
    float4* xr = reinterpret_cast<float4*>(x + (int64_t)r * d);
    const float4* rr = res ? reinterpret_cast<const float4*>(res + (int64_t)r * d) : nullptr;
    const float4* g4 = reinterpret_cast<const float4*>(gain);
    const int n4 = d >> 2;
    float4 v[kWarpVec];
#pragma unroll
    for (int k = 0; k < kWarpVec; k++) {
        const int i = lane + k * 32;
        if (i < n4) v[k] = xr[i];
    }
    if (rr) {
#pragma unroll
        for (int k = 0; k < kWarpVec; k++) {
            const int i = lane + k * 32;
            if (i < n4) {
                const float4 a = rr[i];
                v[k].x += a.x; v[k].y += a.y; v[k].z += a.z; v[k].w += a.w;
                xr[i] = v[k];
            }
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < kWarpVec; k++)
        if (lane + k * 32 < n4) ss += (v[k].x * v[k].x + v[k].y * v[k].y) + (v[k].z * v[k].z + v[k].w * v[k].w);
    ss = warp_sum(ss);
    const float scale = rsqrtf(ss / (float)d + eps);
    uint2* orow = reinterpret_cast<uint2*>(out + (int64_t)r * d);
#pragma unroll
    for (int k = 0; k < kWarpVec; k++) {
        const int i = lane + k * 32;
        if (i < n4) {
            const float4 g = g4[i];
            __nv_bfloat162 lo = __floats2bfloat162_rn(v[k].x * scale * g.x, v[k].y * scale * g.y);
            __nv_bfloat162 hi = __floats2bfloat162_rn(v[k].z * scale * g.z, v[k].w * scale * g.w);
            uint2 pk;
            pk.x = *reinterpret_cast<uint32_t*>(&lo);
            pk.y = *reinterpret_cast<uint32_t*>(&hi);
            orow[i] = pk;
        }
    }
}

// x[r,:] += y[r,:] * rsqrt(mean(y^2) + eps) * gain (a norm on a sublayer's OUTPUT before it
// joins the residual stream), and, with `out`, out[r,:] = x[r,:] * rsqrt(mean(x^2) + eps2) *
// gain2 of the updated row: the norm in front of the next sublayer, in the same pass.
// One block per row; the block size follows from the width, so the order of a row's
// additions does too.
template <typename T>
__global__ void __launch_bounds__(kThreads)
rmsnorm_add_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ gain, float eps,
                   T* __restrict__ out, const float* __restrict__ gain2, float eps2, int d) {
    __shared__ float red[32];
    griddep_wait();
    griddep_launch();
    const int r = blockIdx.x;
    float* xr = x + (int64_t)r * d;
    const float* yr = y + (int64_t)r * d;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) ss += yr[i] * yr[i];
    ss = block_sum(ss, red);
    const float scale = rsqrtf(ss / (float)d + eps);
    float s2 = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        const float v = xr[i] + yr[i] * scale * gain[i];
        xr[i] = v;
        s2 += v * v;
    }
    if (out == nullptr) return;
    T* orow = out + (int64_t)r * d;
    if (gain2 == nullptr) {
        // no norm in front of the next sublayer: it reads the updated rows themselves, in its element type
        for (int i = threadIdx.x; i < d; i += blockDim.x) orow[i] = from_f32<T>(xr[i]);
        return;
    }
    s2 = block_sum(s2, red);
    const float scale2 = rsqrtf(s2 / (float)d + eps2);
    for (int i = threadIdx.x; i < d; i += blockDim.x) orow[i] = from_f32<T>(xr[i] * scale2 * gain2[i]);
}

// Layer norm with gain and bias, the residual sum folded in as in add_rmsnorm_kernel:
//
//   x[r,:] (+)= res[r,:]
//   out[r,:] = (x[r,:] - mean) * rsqrt(var + eps) * gain[:] + bias[:]
//
// mean and var (the mean of the squared deviations, taken about the mean in a second pass)
// are float32.  One block per row whose size follows from the width alone, so a row's sums
// have the same order whatever else the launch holds.  rows as in add_rmsnorm_kernel.
template <typename T, typename R>
__global__ void __launch_bounds__(kThreads)
add_layernorm_kernel(float* __restrict__ x, const R* __restrict__ res, T* __restrict__ out,
                     const float* __restrict__ gain, const float* __restrict__ bias, const int* __restrict__ rows,
                     int d, float eps) {
    __shared__ float red[32];
    griddep_wait();
    griddep_launch();
    const int r = blockIdx.x;
    const int64_t src = rows ? (int64_t)rows[r] : (int64_t)r;
    float* xr = x + src * d;
    const R* rr = res ? res + src * d : nullptr;
    T* orow = out + (int64_t)r * d;
    const bool write_back = (rows == nullptr) && (res != nullptr);
    float sum = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float v = xr[i];
        if (rr) {
            v += to_f32(rr[i]);
            if (write_back) xr[i] = v;
        }
        sum += v;
    }
    const float mean = block_sum(sum, red) / (float)d;
    float sq = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float v = xr[i];
        if (rr && !write_back) v += to_f32(rr[i]);
        v -= mean;
        sq += v * v;
    }
    const float scale = rsqrtf(block_sum(sq, red) / (float)d + eps);
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float v = xr[i];
        if (rr && !write_back) v += to_f32(rr[i]);
        orow[i] = from_f32<T>((v - mean) * scale * gain[i] + bias[i]);
    }
}

// The common case of a step's rows (float32 residual or none, width a multiple of 4 up
// to kThreads * 4 * kVec; every row, or the rows that `rows` names, which are then left as they are) in one
// pass over the memory: a thread keeps its elements in registers
// between the sum, the sum of squared deviations and the scaling, 16-byte accesses.  Whether this
// kernel runs is decided by the width and the addresses alone, never by the number of rows.
template <typename T>
__global__ void __launch_bounds__(kThreads)
add_layernorm_vec4_kernel(float* __restrict__ x, const float* __restrict__ res, T* __restrict__ out,
                          const float* __restrict__ gain, const float* __restrict__ bias,
                          const int* __restrict__ rows, int d, float eps) {
    __shared__ float red[32];
    griddep_wait();
    griddep_launch();
    const int r = blockIdx.x;
    const int64_t src = rows ? (int64_t)rows[r] : (int64_t)r;
    float4* xr = reinterpret_cast<float4*>(x + src * d);
    const float4* rr = res ? reinterpret_cast<const float4*>(res + src * d) : nullptr;
    const float4* g4 = reinterpret_cast<const float4*>(gain);
    const float4* b4 = reinterpret_cast<const float4*>(bias);
    const int n4 = d >> 2;
    float4 v[kVec];
    float sum = 0.f;
#pragma unroll
    for (int k = 0; k < kVec; k++) {
        const int i = threadIdx.x + k * kThreads;
        if (i < n4) {
            v[k] = xr[i];
            if (rr) {
                const float4 a = rr[i];
                v[k].x += a.x; v[k].y += a.y; v[k].z += a.z; v[k].w += a.w;
                if (!rows) xr[i] = v[k];
            }
            sum += (v[k].x + v[k].y) + (v[k].z + v[k].w);
        }
    }
    const float mean = block_sum(sum, red) / (float)d;
    float sq = 0.f;
#pragma unroll
    for (int k = 0; k < kVec; k++) {
        const int i = threadIdx.x + k * kThreads;
        if (i < n4) {
            v[k].x -= mean; v[k].y -= mean; v[k].z -= mean; v[k].w -= mean;
            sq += (v[k].x * v[k].x + v[k].y * v[k].y) + (v[k].z * v[k].z + v[k].w * v[k].w);
        }
    }
    const float scale = rsqrtf(block_sum(sq, red) / (float)d + eps);
#pragma unroll
    for (int k = 0; k < kVec; k++) {
        const int i = threadIdx.x + k * kThreads;
        if (i < n4) {
            const float4 g = g4[i], b = b4[i];
            const float o0 = v[k].x * scale * g.x + b.x, o1 = v[k].y * scale * g.y + b.y;
            const float o2 = v[k].z * scale * g.z + b.z, o3 = v[k].w * scale * g.w + b.w;
            if (sizeof(T) == 4) {
                reinterpret_cast<float4*>(out + (int64_t)r * d)[i] = make_float4(o0, o1, o2, o3);
            } else {
                __nv_bfloat162 lo = __floats2bfloat162_rn(o0, o1);
                __nv_bfloat162 hi = __floats2bfloat162_rn(o2, o3);
                uint2 pk;
                pk.x = *reinterpret_cast<uint32_t*>(&lo);
                pk.y = *reinterpret_cast<uint32_t*>(&hi);
                reinterpret_cast<uint2*>(out + (int64_t)r * d)[i] = pk;
            }
        }
    }
}

}  // namespace

// x float32 [n][d] (updated), y float32 [n][d], gain float32 [d]; out (optional, element type
// `dtype`) [n][d] with gain2 [d]; gain2 NULL: out gets the updated rows as they are, in its element type.
extern "C" int kllm_rmsnorm_add(void* x, const void* y, const void* gain, float eps, void* out, const void* gain2,
                                float eps2, int n_rows, int d, int dtype, void* stream) {
    if (n_rows <= 0) return 0;
    if (d <= 0) KLLM_FAIL("rmsnorm_add: width %d must be positive", d);
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = d <= 512 ? 64 : (d <= 2048 ? 128 : kThreads);
    if (dtype == KLLM_F32)
        kllm_launch((rmsnorm_add_kernel<float>), dim3(n_rows), dim3(threads), 0, s, (float*)x, (const float*)y,
                    (const float*)gain, eps, (float*)out, (const float*)gain2, eps2, d);
    else if (dtype == KLLM_BF16)
        kllm_launch((rmsnorm_add_kernel<bf16>), dim3(n_rows), dim3(threads), 0, s, (float*)x, (const float*)y,
                    (const float*)gain, eps, (bf16*)out, (const float*)gain2, eps2, d);
    else
        KLLM_FAIL("rmsnorm_add: unknown element type %d", dtype);
    KLLM_LAUNCH_STATUS();
}

// dtype: element type of out; res_dtype: element type of res (ignored when res is NULL).
extern "C" int kllm_add_rmsnorm(void* x, const void* res, void* out, const void* gain,
                                const int* rows, int n_rows, int d, float eps, int dtype,
                                int res_dtype, void* stream) {
    if (n_rows <= 0) return 0;
    if (d <= 0) KLLM_FAIL("rmsnorm: width %d must be positive", d);
    cudaStream_t s = (cudaStream_t)stream;
    auto aligned = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
    if (dtype == KLLM_BF16 && (res == nullptr || res_dtype == KLLM_F32) && rows == nullptr && (d & 3) == 0 &&
        d <= kThreads * 4 * kVec && aligned(x) && aligned(res) && aligned(gain) && ((uintptr_t)out & 7) == 0) {
        if (d <= 32 * 4 * kWarpVec) {
            kllm_launch((add_rmsnorm_warp_kernel), dim3((n_rows + 7) / 8), dim3(256), 0, s, (float*)x, (const float*)res,
                        (bf16*)out, (const float*)gain, n_rows, d, eps);
            KLLM_LAUNCH_STATUS();
        }
        kllm_launch((add_rmsnorm_vec4_kernel), dim3(n_rows), dim3(kThreads), 0, s, (float*)x, (const float*)res, (bf16*)out,
                    (const float*)gain, d, eps);
        KLLM_LAUNCH_STATUS();
    }
    if (res == nullptr) res_dtype = dtype;
    if (dtype == KLLM_F32 && res_dtype == KLLM_F32) {
        kllm_launch((add_rmsnorm_kernel<float, float>), dim3(n_rows), dim3(kThreads), 0, s, 
            (float*)x, (const float*)res, (float*)out, (const float*)gain, rows, d, eps);
    } else if (dtype == KLLM_BF16 && res_dtype == KLLM_BF16) {
        kllm_launch((add_rmsnorm_kernel<bf16, bf16>), dim3(n_rows), dim3(kThreads), 0, s, 
            (float*)x, (const bf16*)res, (bf16*)out, (const float*)gain, rows, d, eps);
    } else if (dtype == KLLM_BF16 && res_dtype == KLLM_F32) {
        kllm_launch((add_rmsnorm_kernel<bf16, float>), dim3(n_rows), dim3(kThreads), 0, s, 
            (float*)x, (const float*)res, (bf16*)out, (const float*)gain, rows, d, eps);
    } else {
        KLLM_FAIL("rmsnorm: element types %d (out) and %d (res) are not supported together", dtype, res_dtype);
    }
    KLLM_LAUNCH_STATUS();
}

// Layer norm with gain and bias (both float32 [d]); the other arguments as in kllm_add_rmsnorm.
extern "C" int kllm_add_layernorm(void* x, const void* res, void* out, const void* gain, const void* bias,
                                  const int* rows, int n_rows, int d, float eps, int dtype, int res_dtype,
                                  void* stream) {
    if (n_rows <= 0) return 0;
    if (d <= 0) KLLM_FAIL("layernorm: width %d must be positive", d);
    if (!gain || !bias) KLLM_FAIL("layernorm: gain and bias are required");
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = d <= 512 ? 64 : (d <= 2048 ? 128 : kThreads);
    auto aligned = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
    if ((res == nullptr || res_dtype == KLLM_F32) && (d & 3) == 0 && d <= kThreads * 4 * kVec &&
        aligned(x) && aligned(res) && aligned(gain) && aligned(bias) && aligned(out) &&
        (dtype == KLLM_BF16 || dtype == KLLM_F32)) {
        if (dtype == KLLM_BF16)
            kllm_launch((add_layernorm_vec4_kernel<bf16>), dim3(n_rows), dim3(kThreads), 0, s, (float*)x, (const float*)res,
                        (bf16*)out, (const float*)gain, (const float*)bias, rows, d, eps);
        else
            kllm_launch((add_layernorm_vec4_kernel<float>), dim3(n_rows), dim3(kThreads), 0, s, (float*)x, (const float*)res,
                        (float*)out, (const float*)gain, (const float*)bias, rows, d, eps);
        KLLM_LAUNCH_STATUS();
    }
    if (res == nullptr) res_dtype = dtype;
#define KLLM_LN(T, R)                                                                                           \
    kllm_launch((add_layernorm_kernel<T, R>), dim3(n_rows), dim3(threads), 0, s, (float*)x, (const R*)res, (T*)out, \
                (const float*)gain, (const float*)bias, rows, d, eps)
    if (dtype == KLLM_F32 && res_dtype == KLLM_F32) KLLM_LN(float, float);
    else if (dtype == KLLM_BF16 && res_dtype == KLLM_BF16) KLLM_LN(bf16, bf16);
    else if (dtype == KLLM_BF16 && res_dtype == KLLM_F32) KLLM_LN(bf16, float);
    else KLLM_FAIL("layernorm: element types %d (out) and %d (res) are not supported together", dtype, res_dtype);
#undef KLLM_LN
    KLLM_LAUNCH_STATUS();
}
