// Routed experts: every token runs `top` of E small gated feed-forwards.
//
//   route     z = W_r h in float32 (h widened from the model's element type), score =
//             sigmoid(z) or softmax(z); the `top` largest scores, the lower index first among
//             equals; the weights are the chosen scores, as they are or divided by their sum.
//             Optionally the experts form equal groups of neighbours, a group scores as its best
//             expert, and only experts of the `keep` best groups can be chosen.
//   sort      the (token, choice) pairs ordered by expert: offsets[E + 1] and perm[n * top]
//             (sorted row -> token * top + choice), on the device, so that a step's launch
//             shapes do not depend on the routing.
//   gemm      for the sorted rows of every expert e, C = A W_e^T with float32 accumulation:
//             bfloat16 operands as tiles of 64 rows x 64 columns on the tensor cores
//             (mma.sync m16n8k16, operands through a three-stage cp.async ring), float32
//             operands (and bfloat16 ones whose rows are not 16-byte aligned) as tiles of 32 x
//             64 on the CUDA cores.  Two forms:
//             "gated" reads row `token` of the layer's input, times the row's weight if the
//             weight acts on the expert's input, and stores act(gate) * up per sorted row;
//             "down" reads the sorted rows and stores row token * top + choice of a float32
//             matrix, times the weight if it acts on the output.
//   combine   y[t] = sum over the choices of a token, in choice order; optionally plus the row of
//             an expert that every token runs, times the sigmoid of a gate logit per token.
//   table     instead of a router: a table [vocab][top] that gives every token id its experts,
//             each with the same weight.
// The gated activation is silu(g) * u, or with a limit L and a slope a the clamped form
// min(g, L) * sigmoid(a min(g, L)) * (clamp(u, -L, L) + 1).
//
// A row's sums do not depend on which other rows share its tile or its launch.
#include "common.cuh"

KLLM_EXPORT_LAST_ERROR(moe)

namespace {

// ---- router ----------------------------------------------------------------------
// one CTA of four warps per token: the warps share the columns of the router's rows, so that a step of
// few tokens still has many loads in flight (the router's rows come from HBM in every decode step: the
// weights streamed between two steps push them out of L2); warp 0 then makes the choice.  E logits in
// shared memory (E <= 1024).  A logit's sum has one order, fixed by the width.
template <typename T>
__global__ void __launch_bounds__(128)
route_kernel(int* __restrict__ idx, float* __restrict__ wt, const T* __restrict__ h, const float* __restrict__ router,
             int n, int d, int E, int top, int softmax, int renorm, int groups, int keep) {
    extern __shared__ float zsh[];            // [E], then [2 * groups] when groups limit the choice
    __shared__ float part[4][8];
    griddep_wait();
    griddep_launch();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = blockIdx.x;
    float* z = zsh;
    const T* hr = h + (int64_t)t * d;
    // eight experts at a time: their loads are independent of one another, and the token's row is read
    // once for all eight; every expert's sum still runs over its columns in the one order
    for (int e0 = 0; e0 < E; e0 += 8) {
        const float* wr[8];
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; j++) {
            wr[j] = router + (int64_t)min(e0 + j, E - 1) * d;
            acc[j] = 0.f;
        }
#pragma unroll 4
        for (int c = threadIdx.x; c < d; c += 128) {
            const float hv = to_f32(hr[c]);
#pragma unroll
            for (int j = 0; j < 8; j++) acc[j] += hv * wr[j][c];
        }
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const float a = warp_sum(acc[j]);
            if (lane == 0) part[warp][j] = a;
        }
        __syncthreads();
        if (threadIdx.x < 8 && e0 + threadIdx.x < E)
            z[e0 + threadIdx.x] = (part[0][threadIdx.x] + part[1][threadIdx.x]) + (part[2][threadIdx.x] + part[3][threadIdx.x]);
        __syncthreads();
    }
    if (warp != 0) return;
    // the choice is made among the logits: both scores grow with them, and a sigmoid that has
    // reached 1.0f no longer tells two experts apart
    float zmax = 0.f, zsum = 1.f;
    if (softmax) {
        zmax = -INFINITY;
        for (int e = lane; e < E; e += 32) zmax = fmaxf(zmax, z[e]);
        zmax = warp_max(zmax);
        zsum = 0.f;
        for (int e = lane; e < E; e += 32) zsum += expf(z[e] - zmax);
        zsum = warp_sum(zsum);
    }
    if (groups > 1 && keep < groups) {
        // The experts form `groups` equal groups of neighbours; a group's score is its best expert's
        // (the logits order as the scores do).  Only experts of the `keep` best groups can be chosen,
        // the lower group first among equals; the scores themselves stay those over all experts.
        float* gb = zsh + E;                              // a group's best logit, then whether it is kept
        const int per = E / groups;
        for (int gi = lane; gi < groups; gi += 32) {
            float b = -INFINITY;
            for (int j = 0; j < per; j++) b = fmaxf(b, z[gi * per + j]);
            gb[gi] = b;
            gb[groups + gi] = 0.f;
        }
        __syncwarp();
        for (int c = 0; c < keep; c++) {
            float best = -INFINITY;
            int bi = groups;
            for (int gi = lane; gi < groups; gi += 32)
                if (gb[groups + gi] == 0.f && (gb[gi] > best || bi == groups)) { best = gb[gi]; bi = gi; }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (oi < groups && (bi == groups || ob > best || (ob == best && oi < bi))) { best = ob; bi = oi; }
            }
            if (lane == 0 && bi < groups) gb[groups + bi] = 1.f;
            __syncwarp();
        }
        for (int e = lane; e < E; e += 32)
            if (gb[groups + e / per] == 0.f) z[e] = -INFINITY;
        __syncwarp();
    }
    float total = 0.f;
    for (int c = 0; c < top; c++) {
        float best = -INFINITY;
        int bi = E;
        for (int e = lane; e < E; e += 32)
            if (z[e] > best) { best = z[e]; bi = e; }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
        }
        const float score = softmax ? expf(best - zmax) / zsum : 1.f / (1.f + expf(-best));
        if (lane == 0) {
            idx[(int64_t)t * top + c] = bi;
            wt[(int64_t)t * top + c] = score;
            z[bi] = -INFINITY;
        }
        total += score;
        __syncwarp();
    }
    if (renorm && lane == 0)
        for (int c = 0; c < top; c++) wt[(int64_t)t * top + c] /= total;
}

// ---- sort by expert ---------------------------------------------------------------
// one CTA; counts and offsets in shared memory.  The order of the rows inside an expert is
// whatever the atomics give: no result depends on it.
__global__ void __launch_bounds__(1024)
sort_kernel(int* __restrict__ offsets, int* __restrict__ perm, int* __restrict__ rank, const int* __restrict__ idx,
            int rows, int E) {
    extern __shared__ int cnt[];              // [E + 1]
    griddep_wait();
    griddep_launch();
    for (int e = threadIdx.x; e <= E; e += blockDim.x) cnt[e] = 0;
    __syncthreads();
    for (int r = threadIdx.x; r < rows; r += blockDim.x) rank[r] = atomicAdd(&cnt[idx[r]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int e = 0; e < E; e++) {
            const int c = cnt[e];
            cnt[e] = run;
            run += c;
        }
        cnt[E] = run;
    }
    __syncthreads();
    for (int e = threadIdx.x; e <= E; e += blockDim.x) offsets[e] = cnt[e];
    for (int r = threadIdx.x; r < rows; r += blockDim.x) perm[cnt[idx[r]] + rank[r]] = r;
}

// ---- the experts' products ---------------------------------------------------------
constexpr int BM = 32, BN = 64, BK = 32, GT = 256;

__device__ __forceinline__ float act_silu(float g) { return g / (1.f + expf(-g)); }

// The gated activation of an expert.  kind 0: silu(g) * u.  kind 1, with a limit L and a
// slope a: g' = min(g, L), u' = clamp(u, -L, L), g' * sigmoid(a g') * (u' + 1).
struct GatedAct {
    int kind;
    float limit, alpha;
};
__device__ __forceinline__ float gated_act(float g, float u, const GatedAct& a) {
    if (a.kind == 0) return act_silu(g) * u;
    g = fminf(g, a.limit);
    u = fminf(fmaxf(u, -a.limit), a.limit);
    return g / (1.f + expf(-a.alpha * g)) * (u + 1.f);
}

// GATED: W_e is [2 * N][K] (gate rows, then up rows), C [rows][N] in T, sorted order.
// else : W_e is [N][K], C float32 [rows][N] at row perm[r].
template <typename T, bool GATED>
__global__ void __launch_bounds__(GT)
expert_gemm_kernel(void* __restrict__ c_out, const T* __restrict__ a, int64_t a_stride, const T* __restrict__ w,
                   const int* __restrict__ offsets, const int* __restrict__ perm, const float* __restrict__ wt,
                   int E, int top, int N, int K, int scale_in, int scale_out, GatedAct act) {
    __shared__ float As[BK][BM + 1];
    __shared__ float Ws[GATED ? 2 : 1][BK][BN + 1];
    __shared__ int srow[BM];
    __shared__ float sscale[BM];
    griddep_wait();
    griddep_launch();
    // which expert and which of its row tiles
    int tile = blockIdx.y, e = 0, lo = 0, hi = 0;
    for (; e < E; e++) {
        lo = offsets[e];
        hi = offsets[e + 1];
        const int nt = (hi - lo + BM - 1) / BM;
        if (tile < nt) break;
        tile -= nt;
    }
    if (e >= E) return;
    const int r0 = lo + tile * BM, nr = min(BM, hi - r0);
    const int n0 = blockIdx.x * BN;
    const int tid = threadIdx.x;
    if (tid < BM) {
        int src = 0;
        float sc = 1.f;
        if (tid < nr) {
            const int flat = perm[r0 + tid];
            src = GATED ? flat / top : r0 + tid;
            if (GATED ? scale_in : scale_out) sc = wt[flat];
        }
        srow[tid] = src;
        sscale[tid] = sc;
    }
    __syncthreads();
    const T* we = w + (int64_t)e * (GATED ? 2 : 1) * N * K;
    const int ty = tid / 16, tx = tid % 16;                 // rows ty, ty + 16; columns tx + 16 j
    float acc[GATED ? 2 : 1][2][4] = {};
    for (int k0 = 0; k0 < K; k0 += BK) {
        for (int i = tid; i < BM * BK; i += GT) {
            const int rr = i / BK, kk = i - rr * BK;
            float v = 0.f;
            if (rr < nr && k0 + kk < K) {
                v = to_f32(a[(int64_t)srow[rr] * a_stride + k0 + kk]);
                if (GATED) v *= sscale[rr];
            }
            As[kk][rr] = v;
        }
        for (int i = tid; i < BN * BK; i += GT) {
            const int cc = i / BK, kk = i - cc * BK;
            const bool ok = n0 + cc < N && k0 + kk < K;
            Ws[0][kk][cc] = ok ? to_f32(we[(int64_t)(n0 + cc) * K + k0 + kk]) : 0.f;
            if (GATED) Ws[1][kk][cc] = ok ? to_f32(we[(int64_t)(N + n0 + cc) * K + k0 + kk]) : 0.f;
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < BK; kk++) {
            const float a0 = As[kk][ty], a1 = As[kk][ty + 16];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const float b = Ws[0][kk][tx + 16 * j];
                acc[0][0][j] += a0 * b;
                acc[0][1][j] += a1 * b;
                if (GATED) {
                    const float b2 = Ws[1][kk][tx + 16 * j];
                    acc[1][0][j] += a0 * b2;
                    acc[1][1][j] += a1 * b2;
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; i++) {
        const int rr = ty + 16 * i;
        if (rr >= nr) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int cc = n0 + tx + 16 * j;
            if (cc >= N) continue;
            if (GATED) {
                ((T*)c_out)[(int64_t)(r0 + rr) * N + cc] = from_f32<T>(gated_act(acc[0][i][j], acc[GATED ? 1 : 0][i][j], act));
            } else {
                ((float*)c_out)[(int64_t)perm[r0 + rr] * N + cc] = acc[0][i][j] * sscale[rr];
            }
        }
    }
}

// ---- the same on the tensor cores, bfloat16 ---------------------------------------------------
// 256 threads: warp (wm, wn) = (w % 4, w / 4) owns MW 16-row tiles of the rows and columns 32 wn ..
// 32 wn + 31 of the tile's 64.  A weight on
// the expert's input is applied to the accumulators instead: W (s x) = s (W x), the same
// number without rounding s x to bfloat16 first.
constexpr int TN = 64, TK = 64, TLD = TK + 8, TSTAGES = 3, TT = 256;

__device__ __forceinline__ void cp16(bf16* dst, const bf16* src, bool ok) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    const int bytes = ok ? 16 : 0;                          // 0: filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], const bf16* p) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <bool GATED, int MW>
constexpr size_t mma_smem_bytes() {
    return (size_t)TSTAGES * (64 * MW + (GATED ? 2 : 1) * TN) * TLD * sizeof(bf16);
}

// MW: 16-row tiles per warp; a CTA's tile has TM = 64 * MW rows (128 where an expert has many
// rows, so that a weight fragment serves two row tiles; 64 otherwise).
template <bool GATED, int MW>
__global__ void __launch_bounds__(TT)
expert_gemm_mma_kernel(void* __restrict__ c_out, const bf16* __restrict__ a, int64_t a_stride, const bf16* __restrict__ w,
                       const int* __restrict__ offsets, const int* __restrict__ perm, const float* __restrict__ wt,
                       int E, int top, int N, int K, int scale_in, int scale_out, GatedAct act) {
    constexpr int NB = GATED ? 2 : 1, TM = 64 * MW;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16 (*As)[TM][TLD] = reinterpret_cast<bf16 (*)[TM][TLD]>(smem_raw);                           // [TSTAGES]
    bf16 (*Bs)[NB][TN][TLD] = reinterpret_cast<bf16 (*)[NB][TN][TLD]>(smem_raw + (size_t)TSTAGES * TM * TLD * sizeof(bf16));
    __shared__ int srow[TM];
    __shared__ int sdst[TM];
    __shared__ float sscale[TM];
    griddep_wait();
    griddep_launch();
    int tile = blockIdx.y, e = 0, lo = 0, hi = 0;
    for (; e < E; e++) {
        lo = offsets[e];
        hi = offsets[e + 1];
        const int nt = (hi - lo + TM - 1) / TM;
        if (tile < nt) break;
        tile -= nt;
    }
    if (e >= E) return;
    const int r0 = lo + tile * TM, nr = min(TM, hi - r0), n0 = blockIdx.x * TN;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gid = lane >> 2, tq = lane & 3;
    const int wm = warp & 3, wn = warp >> 2;
    for (int i = tid; i < TM; i += TT) {
        int src = 0, dst = 0;
        float sc = 1.f;
        if (i < nr) {
            const int flat = perm[r0 + i];
            src = GATED ? flat / top : r0 + i;
            dst = flat;
            if (GATED ? scale_in : scale_out) sc = wt[flat];
        }
        srow[i] = src;
        sdst[i] = dst;
        sscale[i] = sc;
    }
    __syncthreads();
    const bf16* we = w + (int64_t)e * NB * N * K;
    auto load = [&](int stage, int k0) {
        // rows x 8 chunks of 8 elements, for A and for each weight tile
        for (int i = tid; i < TM * (TK / 8); i += TT) {
            const int rr = i / (TK / 8), ch = (i % (TK / 8)) * 8;
            const bool ok = rr < nr && k0 + ch < K;
            cp16(&As[stage][rr][ch], a + (ok ? (int64_t)srow[rr] * a_stride + k0 + ch : 0), ok);
        }
#pragma unroll
        for (int b = 0; b < NB; b++)
            for (int i = tid; i < TN * (TK / 8); i += TT) {
                const int cc = i / (TK / 8), ch = (i % (TK / 8)) * 8;
                const bool ok = n0 + cc < N && k0 + ch < K;
                cp16(&Bs[stage][b][cc][ch], we + (ok ? ((int64_t)b * N + n0 + cc) * K + k0 + ch : 0), ok);
            }
    };
    float acc[NB][MW][4][4] = {};
    const int nk = (K + TK - 1) / TK;
#pragma unroll
    for (int st = 0; st < TSTAGES - 1; st++) {
        if (st < nk) load(st, st * TK);
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    }
    for (int it = 0; it < nk; it++) {
        asm volatile("cp.async.wait_group %0;\n" ::"n"(TSTAGES - 2) : "memory");
        __syncthreads();
        const int nxt = it + TSTAGES - 1;
        if (nxt < nk) load(nxt % TSTAGES, nxt * TK);
        asm volatile("cp.async.commit_group;\n" ::: "memory");
        const int st = it % TSTAGES;
        if (16 * MW * wm >= nr) continue;                   // none of this warp's rows exists
#pragma unroll
        for (int ks = 0; ks < TK / 16; ks++) {
            uint32_t af[MW][4];
#pragma unroll
            for (int m = 0; m < MW; m++)
                ldsm4(af[m], &As[st][16 * (MW * wm + m) + (lane & 15)][ks * 16 + (lane >> 4) * 8]);
#pragma unroll
            for (int b = 0; b < NB; b++)
#pragma unroll
                for (int np = 0; np < 2; np++) {
                    uint32_t bfr[4];
                    ldsm4(bfr, &Bs[st][b][32 * wn + 16 * np + (lane >> 4) * 8 + (lane & 7)][ks * 16 + ((lane >> 3) & 1) * 8]);
#pragma unroll
                    for (int m = 0; m < MW; m++) {
                        mma16816(acc[b][m][2 * np], af[m], bfr[0], bfr[1]);
                        mma16816(acc[b][m][2 * np + 1], af[m], bfr[2], bfr[3]);
                    }
                }
        }
    }
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
#pragma unroll
    for (int m = 0; m < MW; m++)
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int rr = 16 * (MW * wm + m) + gid + 8 * h;
            if (rr >= nr) continue;
            const float sc = sscale[rr];
#pragma unroll
            for (int nt = 0; nt < 4; nt++)
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    const int cc = n0 + 32 * wn + nt * 8 + 2 * tq + j;
                    if (cc >= N) continue;
                    if (GATED) {
                        const float gv = acc[0][m][nt][2 * h + j] * sc, uv = acc[NB - 1][m][nt][2 * h + j] * sc;
                        ((bf16*)c_out)[(int64_t)(r0 + rr) * N + cc] = __float2bfloat16_rn(gated_act(gv, uv, act));
                    } else {
                        ((float*)c_out)[(int64_t)sdst[rr] * N + cc] = acc[0][m][nt][2 * h + j] * sc;
                    }
                }
        }
}

template <bool GATED, int MW>
int launch_mma(void* c, const void* a, int64_t a_stride, const void* w, const int* offsets, const int* perm,
               const float* wt, int rows, int E, int top, int N, int K, int scale_in, int scale_out, GatedAct act,
               cudaStream_t s) {
    auto kern = expert_gemm_mma_kernel<GATED, MW>;
    static bool raised = false;
    constexpr size_t smem = mma_smem_bytes<GATED, MW>();
    if (!raised) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) {
            snprintf(g_kllm_err, sizeof(g_kllm_err), "moe gemm: shared memory limit: %s", cudaGetErrorString(e));
            return (int)e;
        }
        raised = true;
    }
    const int row_tiles = (rows + 64 * MW - 1) / (64 * MW) + E;
    if (row_tiles > 65535) KLLM_FAIL("moe gemm: %d rows in one launch", rows);
    kllm_launch(kern, dim3((N + TN - 1) / TN, row_tiles), dim3(TT), smem, s, c, (const bf16*)a, a_stride, (const bf16*)w,
                offsets, perm, wt, E, top, N, K, scale_in, scale_out, act);
    KLLM_LAUNCH_STATUS();
}

__global__ void __launch_bounds__(256)
combine_kernel(float* __restrict__ y, const float* __restrict__ parts, int64_t total, int d, int top,
               const float* __restrict__ shared, const float* __restrict__ gate, int64_t gate_stride, float scale) {
    griddep_wait();
    griddep_launch();
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = i / d;
        const int c = (int)(i - t * d);
        float s = 0.f;
        for (int j = 0; j < top; j++) s += parts[(t * top + j) * d + c];
        s *= scale;
        if (shared) s += shared[i] * (gate ? 1.f / (1.f + expf(-gate[t * gate_stride])) : 1.f);
        y[i] = s;
    }
}

// idx[t][j] = table[id of token t][j], wt = weight for every pair: experts that a table gives
// a token by its id.  An id -(s + 1) stands for last_token[s], a choice of the step before that
// is still on the device.
__global__ void __launch_bounds__(256)
table_route_kernel(int* __restrict__ idx, float* __restrict__ wt, const int* __restrict__ token_ids,
                   const int* __restrict__ last_token, const int* __restrict__ table, int n, int vocab, int E, int top,
                   float weight) {
    griddep_wait();
    griddep_launch();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n * top) return;
    const int t = i / top, j = i - t * top;
    int id = token_ids[t];
    if (id < 0 && last_token) id = last_token[-id - 1];
    id = min(max(id, 0), vocab - 1);
    idx[i] = min(max(table[(int64_t)id * top + j], 0), E - 1);
    wt[i] = weight;
}

}  // namespace

// idx int32 [n][top], wt float32 [n][top]; h [n][d] contiguous in `dtype`; router float32 [E][d].
extern "C" int kllm_moe_route(int* idx, float* wt, const void* h, const float* router, int n, int d, int E, int top,
                              int softmax, int renorm, int groups, int keep, int dtype, void* stream) {
    if (n <= 0) return 0;
    if (E <= 0 || E > 1024 || top <= 0 || top > E) KLLM_FAIL("moe route: %d of %d experts (at most 1024)", top, E);
    if (groups < 1) groups = keep = 1;
    if (E % groups || keep < 1 || keep > groups || top > keep * (E / groups))
        KLLM_FAIL("moe route: %d of %d experts in %d groups of which %d are kept", top, E, groups, keep);
    cudaStream_t s = (cudaStream_t)stream;
    const size_t smem = (size_t)(E + 2 * groups) * sizeof(float);
    if (dtype == KLLM_F32)
        kllm_launch((route_kernel<float>), dim3(n), dim3(128), smem, s, idx, wt, (const float*)h, router, n, d, E,
                    top, softmax, renorm, groups, keep);
    else if (dtype == KLLM_BF16)
        kllm_launch((route_kernel<bf16>), dim3(n), dim3(128), smem, s, idx, wt, (const bf16*)h, router, n, d, E,
                    top, softmax, renorm, groups, keep);
    else
        KLLM_FAIL("moe route: unknown element type %d", dtype);
    KLLM_LAUNCH_STATUS();
}

// offsets int32 [E + 1], perm and rank int32 [rows], idx int32 [rows] with values in [0, E).
extern "C" int kllm_moe_sort(int* offsets, int* perm, int* rank, const int* idx, int rows, int E, void* stream) {
    if (rows <= 0) return 0;
    if (E <= 0 || E > 1024) KLLM_FAIL("moe sort: %d experts (at most 1024)", E);
    kllm_launch((sort_kernel), dim3(1), dim3(1024), (size_t)(E + 1) * sizeof(int), (cudaStream_t)stream, offsets, perm, rank,
                idx, rows, E);
    KLLM_LAUNCH_STATUS();
}

// gated != 0: a [tokens][K] (row stride a_stride), w [E][2N][K], c [rows][N] in `dtype`;
// gated == 0: a [rows][K] sorted, w [E][N][K], c float32 [rows][N] indexed by perm.
extern "C" int kllm_moe_gemm(void* c, const void* a, int64_t a_stride, const void* w, const int* offsets,
                             const int* perm, const float* wt, int rows, int E, int top, int N, int K, int gated,
                             int scale_in, int scale_out, int act_kind, float act_limit, float act_alpha, int dtype,
                             void* stream) {
    if (rows <= 0) return 0;
    if (N <= 0 || K <= 0 || E <= 0 || top <= 0) KLLM_FAIL("moe gemm: bad sizes");
    if (act_kind < 0 || act_kind > 1) KLLM_FAIL("moe gemm: unknown activation %d", act_kind);
    const GatedAct act = {act_kind, act_limit, act_alpha};
    const int row_tiles = (rows + BM - 1) / BM + E;
    if (row_tiles > 65535) KLLM_FAIL("moe gemm: %d rows in one launch", rows);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == KLLM_BF16 && K % 8 == 0 && a_stride % 8 == 0 && (((uintptr_t)a | (uintptr_t)w) & 15) == 0) {
        // tiles of 128 rows where the experts have that many rows on average (which tile a row
        // falls into changes no sum of that row)
        const bool tall = rows / E >= 128;
#define KLLM_MOE_MMA(G, MW) \
    return launch_mma<G, MW>(c, a, a_stride, w, offsets, perm, wt, rows, E, top, N, K, scale_in, scale_out, act, s)
        if (gated && tall) KLLM_MOE_MMA(true, 2);
        if (gated) KLLM_MOE_MMA(true, 1);
        if (tall) KLLM_MOE_MMA(false, 2);
        KLLM_MOE_MMA(false, 1);
#undef KLLM_MOE_MMA
    }
    const dim3 grid((N + BN - 1) / BN, row_tiles);
#define KLLM_MOE(T, G)                                                                                            \
    kllm_launch((expert_gemm_kernel<T, G>), grid, dim3(GT), 0, s, c, (const T*)a, a_stride, (const T*)w, offsets, perm, \
                wt, E, top, N, K, scale_in, scale_out, act)
    if (dtype == KLLM_F32) {
        if (gated) KLLM_MOE(float, true); else KLLM_MOE(float, false);
    } else if (dtype == KLLM_BF16) {
        if (gated) KLLM_MOE(bf16, true); else KLLM_MOE(bf16, false);
    } else {
        KLLM_FAIL("moe gemm: unknown element type %d", dtype);
    }
#undef KLLM_MOE
    KLLM_LAUNCH_STATUS();
}

// table int32 [vocab][top] with values in [0, E); token_ids int32 [n]; last_token optional.
extern "C" int kllm_moe_table_route(int* idx, float* wt, const int* token_ids, const int* last_token, const int* table,
                                    int n, int vocab, int E, int top, float weight, void* stream) {
    if (n <= 0) return 0;
    if (vocab <= 0 || E <= 0 || top <= 0 || top > E) KLLM_FAIL("moe table route: %d of %d experts, %d ids", top, E, vocab);
    kllm_launch((table_route_kernel), dim3((n * top + 255) / 256), dim3(256), 0, (cudaStream_t)stream, idx, wt, token_ids,
                last_token, table, n, vocab, E, top, weight);
    KLLM_LAUNCH_STATUS();
}

// y[t] = scale * (sum of parts[t * top + j] over j in order) (+ shared[t] * sigmoid(gate[t * gate_stride]) when
// `shared` float32 [n][d] is given; gate NULL: the shared rows are added as they are).
extern "C" int kllm_moe_combine(float* y, const float* parts, int n, int d, int top, const float* shared,
                                const float* gate, int64_t gate_stride, float scale, void* stream) {
    if (n <= 0) return 0;
    const int64_t total = (int64_t)n * d;
    int64_t blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    kllm_launch((combine_kernel), dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, y, parts, total, d, top,
                shared, gate, gate_stride, scale);
    KLLM_LAUNCH_STATUS();
}
