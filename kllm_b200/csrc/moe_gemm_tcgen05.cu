// The experts' products of a large step on the fifth-generation tensor cores.
//
// The (token, choice) pairs of a step are sorted by expert (moe.cu: offsets[E + 1], perm[rows]);
// expert e owns the sorted rows offsets[e] .. offsets[e + 1].  For those rows C = A W_e^T with
// bfloat16 operands and float32 accumulation, in two forms:
//
//   gated   A [rows, K] is the layer's input gathered into sorted order (gather kernel below),
//           W [E, 2N, K] holds every expert's gate rows and then its up rows; the result
//           act(gate) * up is stored as bfloat16 [rows, N] in sorted order;
//   down    A [rows, K] is that result, W [E, N, K]; the float32 result of sorted row r goes to
//           row perm[r] = token * top + choice of C [rows, N], times the pair's weight if the
//           weights act on the experts' outputs.
//
// The kernel is the persistent one of gemm_tcgen05.cu (a TMA producer warp, a warp that issues
// tcgen05.mma into two accumulators in tensor memory, eight epilogue warps, every wait bounded)
// with another map from tile numbers to work: the tiles of 128 rows are counted expert by expert
// from the offsets on the device, so the launch does not depend on the routing.  A tile of an
// expert's last rows also loads the rows after them (the next expert's, or zeros past the end);
// their results are not stored.  In the same way a tile of an expert's last columns loads rows of
// the next expert's matrix and drops those columns.  A row's sums run over k in one fixed order
// and do not depend on which rows share its tile.
#include "common.cuh"

KLLM_EXPORT_LAST_ERROR(moe_gemm_tcgen05)

#include "tc5_common.cuh"

namespace {

constexpr int BM = 128;
constexpr int BK = TC5_BK;
constexpr int THREADS = 320;
constexpr int EPI_THREADS = 256;
constexpr int A_BYTES = BM * 128;
constexpr int MAX_BN = 256;
constexpr int TMEM_COLS = 2 * MAX_BN;
constexpr int MAX_STAGES = 8;
constexpr int SMEM_BYTES = 1024 + 4 * (A_BYTES + MAX_BN * 128);
constexpr int MAX_EXPERTS = 512;

struct GatedAct {
    int kind;            // 0: silu(g) * u; 1: clamped, g' = min(g, limit), u' = clamp(u, -limit, limit): g' sigmoid(alpha g') (u' + 1)
    float limit, alpha;
};
__device__ __forceinline__ float gated_act(float g, float u, const GatedAct& a) {
    if (a.kind == 0) return silu_mul(g, u);
    g = fminf(g, a.limit);
    u = fminf(fmaxf(u, -a.limit), a.limit);
    return g / (1.f + expf(-a.alpha * g)) * (u + 1.f);
}

// expert of row tile gm: first[e] <= gm < first[e + 1] (first: prefix sums of the experts' tile counts)
__device__ __forceinline__ int expert_of(const int* first, int E, int gm) {
    int lo = 0, hi = E - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (first[mid] <= gm) lo = mid; else hi = mid - 1;
    }
    return lo;
}

// rows of x [tokens, K] into sorted order: xs[r] = x[perm[r] / top], 16 bytes per thread and step
__global__ void __launch_bounds__(256)
gather_sorted_kernel(bf16* __restrict__ xs, const bf16* __restrict__ x, int64_t x_stride, const int* __restrict__ perm,
                     int rows, int top, int K) {
    griddep_wait();
    griddep_launch();
    const int per_row = K / 8;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < (int64_t)rows * per_row;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int r = (int)(i / per_row), c = (int)(i - (int64_t)r * per_row) * 8;
        const int t = perm[r] / top;
        *reinterpret_cast<uint4*>(xs + (int64_t)r * K + c) = *reinterpret_cast<const uint4*>(x + (int64_t)t * x_stride + c);
    }
}

template <bool GATED>
__global__ void __launch_bounds__(THREADS, 1)
moe_tc5_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               void* __restrict__ y, const int* __restrict__ offsets, const int* __restrict__ perm,
               const float* __restrict__ wt, int E, int N, int K, int bn, int stages, int scale_out, GatedAct act,
               int* status) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bar_full[MAX_STAGES], bar_empty[MAX_STAGES], bar_acc_full[2], bar_acc_empty[2];
    __shared__ unsigned s_tmem;
    __shared__ int s_abort;
    __shared__ int s_first[MAX_EXPERTS + 1], s_off[MAX_EXPERTS + 1];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int nout = GATED ? bn / 2 : bn;                  // output columns of a tile
    const int w_rows = GATED ? 2 * N : N;                  // rows of one expert's matrix
    const int b_bytes = bn * 128, stage_bytes = A_BYTES + b_bytes;
    const int n_tiles = (N + nout - 1) / nout;
    const int kblocks = (K + BK - 1) / BK;
    volatile int* abort_flag = &s_abort;

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; s++) { mbar_init(&bar_full[s], 1); mbar_init(&bar_empty[s], 1); }
        for (int a = 0; a < 2; a++) { mbar_init(&bar_acc_full[a], 1); mbar_init(&bar_acc_empty[a], EPI_THREADS); }
        s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&s_tmem)), "r"(TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
    }
    // the offsets come from the kernel before this one
    griddep_wait();
    for (int e = threadIdx.x; e <= E; e += THREADS) s_off[e] = offsets[e];
    __syncthreads();
    if (threadIdx.x == 0) {
        int t = 0;
        for (int e = 0; e < E; e++) {
            s_first[e] = t;
            t += (s_off[e + 1] - s_off[e] + BM - 1) / BM;
        }
        s_first[E] = t;
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem = s_tmem;
    const int m_tiles = s_first[E];
    const int tiles = m_tiles * n_tiles;
    griddep_launch();

    if (warp == 0) {
        // ---- producer ----------------------------------------------------------
        if (lane == 0) {
            prefetch_map(&map_a);
            prefetch_map(&map_b);
        }
        int s = 0;
        unsigned ph = 0;
        int issued = 0;
        bool ok = true;
        for (int tile = blockIdx.x; ok && tile < tiles; tile += gridDim.x) {
            const int gm = tile % m_tiles, n0 = (tile / m_tiles) * nout;
            const int e = expert_of(s_first, E, gm);
            const int row0 = s_off[e] + (gm - s_first[e]) * BM;
            const int wrow = e * w_rows + n0;
            for (int kb = 0; kb < kblocks; kb++) {
                ok = mbar_wait(&bar_empty[s], ph ^ 1u, abort_flag, status, 1);
                if (!ok) break;
                if (lane == 0) {
                    const unsigned a = base + (unsigned)(s * stage_bytes), b = a + A_BYTES;
                    mbar_expect_tx(&bar_full[s], (unsigned)stage_bytes);
                    tma_load_2d(a, &map_a, kb * BK, row0, &bar_full[s]);
                    tma_load_2d(b, &map_b, kb * BK, wrow, &bar_full[s]);
                    if (GATED) tma_load_2d(b + (unsigned)(b_bytes / 2), &map_b, kb * BK, wrow + N, &bar_full[s]);
                }
                __syncwarp();
                issued++;
                if (++s == stages) { s = 0; ph ^= 1u; }
            }
        }
        if (!ok || *abort_flag) {
            // copies still in flight must land before the shared memory goes away
            const int back = issued < stages ? issued : stages;
            for (int j = 0; j < back; j++) {
                int sj = s - 1 - j;
                unsigned pj = ph;
                if (sj < 0) { sj += stages; pj ^= 1u; }
                const long long t0 = clock64();
                while (!mbar_try_wait(&bar_full[sj], pj) && clock64() - t0 < kCycleLimit) {}
            }
        }
    } else if (warp == 1) {
        // ---- tensor-core issuer ------------------------------------------------
        const uint32_t idesc = make_idesc(BM, bn);
        int s = 0, acc = 0;
        unsigned ph = 0, acc_ph = 0;
        bool ok = true;
        for (int tile = blockIdx.x; ok && tile < tiles; tile += gridDim.x) {
            ok = mbar_wait(&bar_acc_empty[acc], acc_ph ^ 1u, abort_flag, status, 2);
            if (!ok) break;
            tc_fence_after();
            const unsigned d = tmem + (unsigned)(acc * MAX_BN);
            for (int kb = 0; kb < kblocks; kb++) {
                ok = mbar_wait(&bar_full[s], ph, abort_flag, status, 3);
                if (!ok) break;
                tc_fence_after();
                if (lane == 0) {
                    const unsigned a = base + (unsigned)(s * stage_bytes), b = a + A_BYTES;
#pragma unroll
                    for (int kk = 0; kk < BK / 16; kk++)
                        umma(d, make_desc(a + kk * 32), make_desc(b + kk * 32), idesc, kb > 0 || kk > 0);
                    umma_commit(&bar_empty[s]);
                }
                __syncwarp();
                if (++s == stages) { s = 0; ph ^= 1u; }
            }
            if (!ok) break;
            if (lane == 0) umma_commit(&bar_acc_full[acc]);
            __syncwarp();
            acc ^= 1;
            if (acc == 0) acc_ph ^= 1u;
        }
    } else {
        // ---- epilogue ----------------------------------------------------------
        const int quarter = warp & 3;                      // the 32 lanes of tensor memory this warp may read
        const int half = (warp - 2) >> 2;                  // which half of the tile's 32-column chunks
        const unsigned lane_base = (unsigned)(quarter * 32) << 16;
        const int chunks = (nout + 31) / 32;
        const int c_lo = half == 0 ? 0 : (chunks + 1) / 2, c_hi = half == 0 ? (chunks + 1) / 2 : chunks;
        int acc = 0;
        unsigned acc_ph = 0;
        for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
            const int gm = tile % m_tiles, n0 = (tile / m_tiles) * nout;
            const int e = expert_of(s_first, E, gm);
            const int row = s_off[e] + (gm - s_first[e]) * BM + quarter * 32 + lane;
            const bool row_ok = row < s_off[e + 1];
            const int limit = min(N, n0 + nout);
            int dst = row;
            float sc = 1.f;
            if (!GATED && row_ok) {
                dst = perm[row];
                if (scale_out) sc = wt[dst];
            }
            if (!mbar_wait(&bar_acc_full[acc], acc_ph, abort_flag, status, 4)) break;
            tc_fence_after();
            const unsigned t = tmem + lane_base + (unsigned)(acc * MAX_BN);
#pragma unroll 1
            for (int c = c_lo; c < c_hi; c++) {
                float v[32];
                tmem_ld32(t + c * 32, v);
                if (GATED) {
                    float u[32];
                    tmem_ld32(t + bn / 2 + c * 32, u);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; j++) v[j] = gated_act(v[j], u[j], act);
                } else {
                    tmem_ld_wait();
                }
                const int col = n0 + c * 32;
                if (!row_ok || col >= limit) continue;
                if (GATED) {
                    bf16* p = (bf16*)y + (int64_t)dst * N + col;
                    if (col + 32 <= limit) {
#pragma unroll
                        for (int q = 0; q < 4; q++) {
                            uint4 pk;
                            pk.x = pack_bf16(v[8 * q], v[8 * q + 1]);
                            pk.y = pack_bf16(v[8 * q + 2], v[8 * q + 3]);
                            pk.z = pack_bf16(v[8 * q + 4], v[8 * q + 5]);
                            pk.w = pack_bf16(v[8 * q + 6], v[8 * q + 7]);
                            *reinterpret_cast<uint4*>(p + 8 * q) = pk;
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; j++)
                            if (col + j < limit) p[j] = __float2bfloat16_rn(v[j]);
                    }
                } else {
                    float* p = (float*)y + (int64_t)dst * N + col;
                    if (col + 32 <= limit) {
#pragma unroll
                        for (int q = 0; q < 8; q++)
                            *reinterpret_cast<float4*>(p + 4 * q) =
                                make_float4(v[4 * q] * sc, v[4 * q + 1] * sc, v[4 * q + 2] * sc, v[4 * q + 3] * sc);
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; j++)
                            if (col + j < limit) p[j] = v[j] * sc;
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(&bar_acc_empty[acc]);
            acc ^= 1;
            if (acc == 0) acc_ph ^= 1u;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(TMEM_COLS));
}

// Accumulator width: the widest one with the fewest waves of tiles, counted for the largest
// number of row tiles that the routing can give.
int pick_bn(int row_tiles, int N, bool gated) {
    const int sms = sm_count();
    const int step = gated ? 64 : 16;
    long long best = -1;
    int best_bn = MAX_BN;
    for (int bn = MAX_BN; bn >= 64; bn -= step) {
        const int nout = gated ? bn / 2 : bn;
        const long long tiles = (long long)row_tiles * ((N + nout - 1) / nout);
        const long long waves = (tiles + sms - 1) / sms;
        if (best < 0 || waves < best) { best = waves; best_bn = bn; }
    }
    return best_bn;
}

template <bool GATED>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, void* y, const int* offsets, const int* perm, const float* wt,
           int rows, int E, int N, int K, int bn, int scale_out, GatedAct act, int* status, cudaStream_t stream) {
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(moe_tc5_kernel<GATED>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) {
            snprintf(g_kllm_err, sizeof(g_kllm_err), "moe gemm (tcgen05): %d bytes of shared memory refused: %s", SMEM_BYTES,
                     cudaGetErrorString(e));
            return (int)e;
        }
        attr_set = true;
    }
    const int row_tiles = rows / BM + E;                   // >= the sum of the experts' tile counts
    const int nout = GATED ? bn / 2 : bn;
    const long long tiles = (long long)row_tiles * ((N + nout - 1) / nout);
    const int grid = (int)(tiles < sm_count() ? tiles : sm_count());
    int stages = (SMEM_BYTES - 1024) / (A_BYTES + bn * 128);
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    kllm_launch((moe_tc5_kernel<GATED>), dim3(grid), dim3(THREADS), SMEM_BYTES, stream, ma, mb, y, offsets, perm, wt, E, N, K,
                bn, stages, scale_out, act, status);
    KLLM_LAUNCH_STATUS();
}

}  // namespace

// 1 if the kernels take these sizes and addresses, else 0 (the caller then uses the grouped
// mma.sync kernel).
extern "C" int kllm_moe_gemm_tcgen05_fits(const void* a, const void* w, const void* c, int rows, int E, int N, int K,
                                          int gated) {
    if (rows <= 0 || E <= 0 || E > MAX_EXPERTS || N <= 0 || K <= 0) return 0;
    if ((K & 7) || (N & 7)) return 0;                                      // 16-byte rows for TMA and the vector stores
    if (((uintptr_t)a & 15) || ((uintptr_t)w & 15) || ((uintptr_t)c & 15)) return 0;
    if ((long long)E * (gated ? 2 : 1) * N > 0x7fffffffLL) return 0;
    return 1;
}

// xs [rows, K] = x[perm[r] / top], bfloat16.
extern "C" int kllm_moe_gather_sorted(void* xs, const void* x, int64_t x_stride, const int* perm, int rows, int top, int K,
                                      void* stream) {
    if (rows <= 0) return 0;
    if (K <= 0 || (K & 7) || (x_stride & 7) || top <= 0 || ((uintptr_t)xs & 15) || ((uintptr_t)x & 15))
        KLLM_FAIL("moe gather: rows of %d elements (stride %lld) are not whole 16-byte pieces", K, (long long)x_stride);
    const long long work = (long long)rows * (K / 8);
    const int grid = (int)((work + 255) / 256 < 148 * 8 ? (work + 255) / 256 : 148 * 8);
    kllm_launch((gather_sorted_kernel), dim3(grid), dim3(256), 0, (cudaStream_t)stream, (bf16*)xs, (const bf16*)x, x_stride, perm, rows,
                top, K);
    KLLM_LAUNCH_STATUS();
}

// a [rows, K] bfloat16 in sorted order (dense rows), w [E, (gated ? 2 : 1) * N, K] bfloat16 contiguous.
// gated: c bfloat16 [rows, N] in sorted order; else c float32 [rows, N] at row perm[r], times wt[perm[r]]
// when scale_out.  status: device int that a wait which ran out sets (1: producer, 2: accumulator,
// 3: stage, 4: epilogue).
extern "C" int kllm_moe_gemm_tcgen05(void* c, const void* a, const void* w, const int* offsets, const int* perm,
                                     const float* wt, int rows, int E, int N, int K, int gated, int scale_out,
                                     int act_kind, float act_limit, float act_alpha, int* status, void* stream) {
    if (rows <= 0) return 0;
    if (!kllm_moe_gemm_tcgen05_fits(a, w, c, rows, E, N, K, gated))
        KLLM_FAIL("moe gemm (tcgen05): sizes %d rows, %d experts, %d x %d or an address not taken", rows, E, N, K);
    if (act_kind < 0 || act_kind > 1) KLLM_FAIL("moe gemm (tcgen05): unknown activation %d", act_kind);
    const GatedAct act = {act_kind, act_limit, act_alpha};
    const int row_tiles = rows / BM + E;
    const int bn = pick_bn(row_tiles, N, gated != 0);
    CUtensorMap ma, mb;
    int r = tensor_map(&ma, a, K, rows, K, BM);
    if (r) return r;
    r = tensor_map(&mb, w, K, E * (gated ? 2 : 1) * N, K, gated ? bn / 2 : bn);
    if (r) return r;
    cudaStream_t s = (cudaStream_t)stream;
    if (gated) return launch<true>(ma, mb, c, offsets, perm, wt, rows, E, N, K, bn, scale_out, act, status, s);
    return launch<false>(ma, mb, c, offsets, perm, wt, rows, E, N, K, bn, scale_out, act, status, s);
}
