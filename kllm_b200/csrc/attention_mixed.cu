// Attention whose scores are mixed across the heads before the softmax, over a paged cache, for mixed
// batches of prompt portions and single tokens.
//
// With H query heads on G key/value heads (head h reads kv head h / (H / G)), a matrix M [H][H], a
// window W (0: none) and optional sinks:
//
//     raw_g(i, j)   = scale * q_g(i) . k_kv(g)(j)                  for every head g
//     s_h(i, j)     = sum over g of M[h][g] raw_g(i, j)            the mixing, before mask and softmax
//     visible       : j <= i and (W == 0 or i - j < W)
//     p_h(i, j)     = exp(s_h(i, j)) / (exp(sink_h) + sum over visible j' of exp(s_h(i, j')))
//     out_h(i)      = sum over visible j of p_h(i, j) v_kv(h)(j)
//
// (without sinks the first term of the denominator is absent).  Since every head's score needs all
// heads' raw scores, a CTA holds ALL heads of a tile of query rows: it walks the visible keys in tiles,
// forms the raw scores of all heads for the tile, mixes them, and keeps a running maximum, denominator
// and output per (head, row) as in any streaming softmax.  Scores, mixing, weights and sums are float32
// in both element types; queries, keys and values are widened when they are brought into shared memory.
// The sums of a row run over the keys in ascending order in tiles that start at the first key its
// tile's first row sees, so a row's result depends on how its prompt was cut only through the order of
// float32 additions.
//
// Work per key tile, all in shared memory:  (1) K tile in;  (2) raw scores, a thread per (kv head, row,
// key) computing the scores of that kv head's query heads with one pass over the key;  (3) V tile in over the
// K tile, and the mixing, a thread per (four heads, row, key);  (4) one warp per (head, row): maximum,
// weights, denominator;  (5) the output, a thread per (head, value channel) for all rows of the tile.
#include "common.cuh"

KLLM_EXPORT_LAST_ERROR(attention_mixed)

namespace {

constexpr int kThreads = 256;
constexpr int kMaxPer = 4;      // query heads on a kv head that one thread scores together (a larger group in turns)
constexpr int kMaxTQ = 8;       // rows of a tile

struct Shape {
    int H, G, dk, dv, TQ, TK;
};

__host__ __device__ inline size_t smem_floats(const Shape& s) {
    const size_t kv = (size_t)s.TK * (size_t)((s.G * s.dk > s.G * s.dv ? s.G * s.dk : s.G * s.dv) + 1);
    return (size_t)s.TQ * s.H * s.dk            // q
           + 2 * (size_t)s.TK                   // where each key of the tile lies (a 64-bit offset)
           + (size_t)s.H * s.H                  // M
           + kv                                 // K tile, then V tile
           + 2 * (size_t)s.H * s.TQ * s.TK      // raw, mixed / weights
           + 3 * (size_t)s.H * s.TQ             // maximum, denominator, correction
           + (size_t)s.TQ * s.H * s.dv;         // output
}

// Where the keys j0 .. j0 + TK - 1 of a request lie: (page * G * page_size + slot), the row of kv head 0 in units of
// rows, or -1 past the last key or without a page.  One look-up per key and tile, before the loads that use it.
__device__ __forceinline__ void locate_keys(long long* where, const int* table, int j0, int nk, int TK, int G,
                                            int page_size) {
    for (int jj = threadIdx.x; jj < TK; jj += kThreads) {
        long long w = -1;
        if (jj < nk) {
            const int pos = j0 + jj, lp = pos / page_size;
            const long long page = table[lp];
            if (page >= 0) w = page * G * page_size + (pos - lp * page_size);
        }
        where[jj] = w;
    }
}

// A tile of keys or values into shared memory as float32: dst[jj][g * size + d] at row pitch `pitch`, from a store
// [pages][G][page_size][size]; rows that `where` marks absent are zero.  bfloat16 rows in whole 16-byte pieces are
// read as such.
template <typename T>
__device__ __forceinline__ void load_rows(float* dst, int pitch, const T* __restrict__ cache, const long long* where, int nk,
                                          int G, int size, int page_size) {
    const int w = G * size;
    if (sizeof(T) == 2 && size % 8 == 0) {
        const int w8 = w / 8, s8 = size / 8;
        for (int i = threadIdx.x; i < nk * w8; i += kThreads) {
            const int jj = i / w8, c = i - jj * w8, g = c / s8, d = (c - g * s8) * 8;
            float* o = dst + jj * pitch + g * size + d;
            const long long at = where[jj];
            if (at < 0) {
#pragma unroll
                for (int u = 0; u < 8; u++) o[u] = 0.f;
            } else {
                const uint4 v = *reinterpret_cast<const uint4*>(cache + (at + (long long)g * page_size) * size + d);
                const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    const float2 f = __bfloat1622float2(h[u]);
                    o[2 * u] = f.x;
                    o[2 * u + 1] = f.y;
                }
            }
        }
        return;
    }
#pragma unroll 4
    for (int i = threadIdx.x; i < nk * w; i += kThreads) {
        const int jj = i / w, c = i - jj * w, g = c / size, d = c - g * size;
        const long long at = where[jj];
        dst[jj * pitch + c] = at < 0 ? 0.f : to_f32(cache[(at + (long long)g * page_size) * size + d]);
    }
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
attention_mixed_kernel(T* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
                       const T* __restrict__ q, int64_t q_stride, const T* __restrict__ kcache,
                       const T* __restrict__ vcache, const float* __restrict__ mix, const float* __restrict__ sinks,
                       const int* __restrict__ q_start, const int* __restrict__ start_pos,
                       const int* __restrict__ block_table, int max_blocks, int n_requests, Shape sh, int page_size,
                       int window, float scale) {
    extern __shared__ float sm[];
    const int H = sh.H, G = sh.G, dk = sh.dk, dv = sh.dv, TQ = sh.TQ, TK = sh.TK;
    const int per = H / G;
    const int kw = G * dk, vw = G * dv;
    const int kp = (kw > vw ? kw : vw) + 1;                 // pitch of the K / V tile: odd, so that keys fall into different banks
    long long* where = reinterpret_cast<long long*>(sm);    // [TK]: where each key of the tile lies
    float* qs = sm + 2 * TK;                                // [TQ][H * dk], scaled
    float* ms = qs + (size_t)TQ * H * dk;                   // [H][H]
    float* kt = ms + H * H;                                 // [TK][kp]
    float* raw = kt + (size_t)TK * kp;                      // [H][TQ][TK]
    float* pr = raw + (size_t)H * TQ * TK;                  // [H][TQ][TK]: mixed scores, then weights
    float* mx = pr + (size_t)H * TQ * TK;                   // [H][TQ]
    float* dn = mx + H * TQ;                                // [H][TQ]
    float* cr = dn + H * TQ;                                // [H][TQ]
    float* acc = cr + H * TQ;                               // [TQ][H * dv]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    for (int i = tid; i < H * H; i += kThreads) ms[i] = mix[i];
    griddep_wait();
    griddep_launch();
    // which request and which of its tiles
    int req = 0, tile = blockIdx.x;
    for (; req < n_requests; req++) {
        const int tiles = (q_start[req + 1] - q_start[req] + TQ - 1) / TQ;
        if (tile < tiles) break;
        tile -= tiles;
    }
    if (req >= n_requests) return;
    const int row0 = q_start[req] + tile * TQ;
    const int nq = min(TQ, q_start[req + 1] - row0);
    const int p0 = start_pos[req] + tile * TQ;              // position of the tile's first row
    int hi = p0 + nq - 1;                                   // last key any row sees
    int lo = window > 0 ? max(0, p0 - window + 1) : 0;
    const int* table = block_table + (int64_t)req * max_blocks;
    // with gridDim.y > 1 (single tokens) the keys are cut into that many ranges of whole tiles, one CTA each; the
    // sink belongs to the first range, and a merging kernel joins the ranges' maxima, denominators and sums
    const int splits = gridDim.y, split = blockIdx.y;
    if (splits > 1) {
        const int chunk = (((hi - lo + 1) + splits - 1) / splits + TK - 1) / TK * TK;
        lo += split * chunk;
        hi = min(hi, lo + chunk - 1);
    }

    for (int i = tid; i < nq * H * dk; i += kThreads) {
        const int r = i / (H * dk), c = i - r * (H * dk);
        qs[i] = to_f32(q[(int64_t)(row0 + r) * q_stride + c]) * scale;
    }
    for (int i = tid; i < H * TQ; i += kThreads) {
        const int h = i / TQ;
        mx[i] = (sinks && split == 0) ? sinks[h] : -INFINITY;
        dn[i] = (sinks && split == 0) ? 1.f : 0.f;
    }
    for (int i = tid; i < TQ * H * dv; i += kThreads) acc[i] = 0.f;

    for (int j0 = lo; j0 <= hi; j0 += TK) {
        const int nk = min(TK, hi - j0 + 1);
        __syncthreads();                                    // the tile before has been used up (and qs, mx, acc are set)
        locate_keys(where, table, j0, nk, TK, G, page_size);
        __syncthreads();
        // (1) keys
        load_rows<T>(kt, kp, kcache, where, nk, G, dk, page_size);
        __syncthreads();
        // (2) raw scores of the query heads of one kv head, for one row and one key
        for (int it = tid; it < G * nq * TK; it += kThreads) {
            const int jj = it % TK, i = (it / TK) % nq, g = it / (TK * nq);
            if (jj >= nk) continue;
            const float* kr = kt + jj * kp + g * dk;
            for (int u0 = 0; u0 < per; u0 += kMaxPer) {
                float a[kMaxPer];
#pragma unroll
                for (int u = 0; u < kMaxPer; u++) a[u] = 0.f;
                const float* qr = qs + (size_t)i * H * dk + (size_t)(g * per + u0) * dk;
                const int nu = min(kMaxPer, per - u0);
                for (int d = 0; d < dk; d++) {
                    const float kv = kr[d];
#pragma unroll
                    for (int u = 0; u < kMaxPer; u++)
                        if (u < nu) a[u] = fmaf(qr[u * dk + d], kv, a[u]);
                }
#pragma unroll
                for (int u = 0; u < kMaxPer; u++)
                    if (u < nu) raw[((g * per + u0 + u) * TQ + i) * TK + jj] = a[u];
            }
        }
        __syncthreads();
        // (3) values over the keys' place; mixing and mask
        load_rows<T>(kt, kp, vcache, where, nk, G, dv, page_size);
        const int hb = (H + 3) / 4;
        for (int it = tid; it < hb * nq * TK; it += kThreads) {
            const int jj = it % TK, i = (it / TK) % nq, h0 = (it / (TK * nq)) * 4;
            const int pos = j0 + jj, pi = p0 + i;
            const bool visible = jj < nk && pos <= pi && (window <= 0 || pi - pos < window);
            float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
            if (visible) {
                const float* m0 = ms + h0 * H;
                const bool b1 = h0 + 1 < H, b2 = h0 + 2 < H, b3 = h0 + 3 < H;
                const float* m1 = b1 ? m0 + H : m0;
                const float* m2 = b2 ? m0 + 2 * H : m0;
                const float* m3 = b3 ? m0 + 3 * H : m0;
                for (int g = 0; g < H; g++) {
                    const float r = raw[(g * TQ + i) * TK + jj];
                    a0 = fmaf(m0[g], r, a0);
                    a1 = fmaf(m1[g], r, a1);
                    a2 = fmaf(m2[g], r, a2);
                    a3 = fmaf(m3[g], r, a3);
                }
            } else {
                a0 = a1 = a2 = a3 = -INFINITY;
            }
            pr[((h0 + 0) * TQ + i) * TK + jj] = a0;
            if (h0 + 1 < H) pr[((h0 + 1) * TQ + i) * TK + jj] = a1;
            if (h0 + 2 < H) pr[((h0 + 2) * TQ + i) * TK + jj] = a2;
            if (h0 + 3 < H) pr[((h0 + 3) * TQ + i) * TK + jj] = a3;
        }
        __syncthreads();
        // (4) one warp per (head, row): maximum, weights, denominator (TK <= 32: a lane per key)
        for (int rw = warp; rw < H * nq; rw += kThreads / 32) {
            const int h = rw / nq, i = rw - h * nq;
            float* row = pr + (h * TQ + i) * TK;
            const float s = lane < TK ? row[lane] : -INFINITY;
            const float m_old = mx[h * TQ + i];
            const float m_new = fmaxf(m_old, warp_max(s));
            const float w = (s == -INFINITY) ? 0.f : expf(s - m_new);       // m_new is finite whenever s is
            const float c = (m_old == -INFINITY) ? 0.f : expf(m_old - m_new);
            const float sum = warp_sum(w);
            if (lane < TK) row[lane] = w;
            if (lane == 0) {
                mx[h * TQ + i] = m_new;
                dn[h * TQ + i] = dn[h * TQ + i] * c + sum;
                cr[h * TQ + i] = c;
            }
        }
        __syncthreads();
        // (5) output: a thread per (head, value channel), all rows of the tile (a single token's one row on its own:
        // the general form would issue the other seven rows' instructions with their predicates off)
        if (nq == 1) {
            for (int it = tid; it < H * dv; it += kThreads) {
                const int h = it / dv, e = it - h * dv;
                const float* vr = kt + (h / per) * dv + e;
                const float* pw = pr + (size_t)h * TQ * TK;
                float a = 0.f, b = 0.f;
                int jj = 0;
                for (; jj + 1 < nk; jj += 2) {
                    a = fmaf(pw[jj], vr[jj * kp], a);
                    b = fmaf(pw[jj + 1], vr[(jj + 1) * kp], b);
                }
                if (jj < nk) a = fmaf(pw[jj], vr[jj * kp], a);
                acc[it] = acc[it] * cr[h * TQ] + (a + b);
            }
            continue;
        }
        for (int it = tid; it < H * dv; it += kThreads) {
            const int h = it / dv, e = it - h * dv;
            const float* vr = kt + (h / per) * dv + e;
            float a[kMaxTQ];
#pragma unroll
            for (int i = 0; i < kMaxTQ; i++) a[i] = 0.f;
            for (int jj = 0; jj < nk; jj++) {
                const float v = vr[jj * kp];
#pragma unroll
                for (int i = 0; i < kMaxTQ; i++)
                    if (i < nq) a[i] = fmaf(pr[(h * TQ + i) * TK + jj], v, a[i]);
            }
#pragma unroll
            for (int i = 0; i < kMaxTQ; i++)
                if (i < nq) {
                    float* o = acc + (size_t)i * H * dv + it;
                    *o = *o * cr[h * TQ + i] + a[i];
                }
        }
    }
    __syncthreads();
    if (splits > 1) {
        // TQ is 1: this range's unnormalised sums, maxima and denominators of the token's heads
        float* po = part_o + ((size_t)row0 * splits + split) * H * dv;
        for (int i = tid; i < H * dv; i += kThreads) po[i] = acc[i];
        float* pm = part_ml + ((size_t)row0 * splits + split) * H * 2;
        for (int h = tid; h < H; h += kThreads) {
            pm[2 * h] = mx[h];
            pm[2 * h + 1] = dn[h];
        }
        return;
    }
    for (int i = tid; i < nq * H * dv; i += kThreads) {
        const int r = i / (H * dv), c = i - r * (H * dv), h = c / dv;
        const float d = dn[h * TQ + r];
        out[(int64_t)(row0 + r) * H * dv + c] = from_f32<T>(d > 0.f ? acc[i] / d : 0.f);
    }
}

// Joins the key ranges of single tokens: out[t][h][:] = sum_s e^(m_s - M) acc_s / sum_s e^(m_s - M) l_s, in range order.
// grid (tokens, heads); a thread per value channel.
template <typename T>
__global__ void __launch_bounds__(128)
attention_mixed_merge_kernel(T* __restrict__ out, const float* __restrict__ part_o, const float* __restrict__ part_ml,
                             int splits, int H, int dv) {
    griddep_wait();
    griddep_launch();
    const int t = blockIdx.x, h = blockIdx.y;
    const float* pm = part_ml + (size_t)t * splits * H * 2 + 2 * h;
    float M = -INFINITY;
    for (int s = 0; s < splits; s++) M = fmaxf(M, pm[(size_t)s * H * 2]);
    float den = 0.f;
    for (int s = 0; s < splits; s++) {
        const float m = pm[(size_t)s * H * 2];
        den = fmaf((m == -INFINITY) ? 0.f : expf(m - M), pm[(size_t)s * H * 2 + 1], den);
    }
    const float inv = den > 0.f ? 1.f / den : 0.f;
    for (int e = threadIdx.x; e < dv; e += blockDim.x) {
        float num = 0.f;
        for (int s = 0; s < splits; s++) {
            const float m = pm[(size_t)s * H * 2];
            const float w = (m == -INFINITY) ? 0.f : expf(m - M);
            num = fmaf(w, part_o[((size_t)t * splits + s) * H * dv + (size_t)h * dv + e], num);
        }
        out[(size_t)t * H * dv + (size_t)h * dv + e] = from_f32<T>(num * inv);
    }
}

// ---- single tokens in bfloat16 ---------------------------------------------------------------------------------
// A decoding step reads every key and value of its window once and has one row a token: what counts is that the
// tiles' loads overlap and that little is done per element loaded.  This form keeps the K and V tiles in shared
// memory as they are stored (bfloat16, copied 16 bytes at a time, both on their way before either is used) and widens
// them where they are used; a CTA takes one token and one range of its keys, as the general form does.
struct DecShape {
    int H, G, dk, dv, TK;
};

struct DecLayout {
    size_t q, mix, k, v, raw, p, stats, acc, where, total;
};

__host__ __device__ inline DecLayout dec_layout(const DecShape& s) {
    DecLayout L;
    size_t o = 0;
    L.where = o;  o += (size_t)s.TK * 8;
    L.q = o;      o += (size_t)s.H * s.dk * 4;
    L.mix = o;    o += (size_t)((s.H + 3) / 4) * s.H * 4 * 4;           // [blocks of four heads][H][4]
    L.k = o;      o += (size_t)s.TK * (s.G * s.dk + 8) * 2;
    L.v = o;      o += (size_t)s.TK * (s.G * s.dv + 8) * 2;
    L.raw = o;    o += (size_t)s.H * (s.TK + 1) * 4;
    L.p = o;      o += (size_t)s.H * (s.TK + 4) * 4;
    L.stats = o;  o += 3 * (size_t)s.H * 4;
    o = (o + 15) / 16 * 16;
    L.acc = o;    o += (size_t)s.H * s.dv * 4;
    L.total = (o + 15) / 16 * 16;
    return L;
}

__device__ __forceinline__ void widen8(const uint4& v, float (&f)[8]) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int u = 0; u < 4; u++) {
        const float2 x = __bfloat1622float2(h[u]);
        f[2 * u] = x.x;
        f[2 * u + 1] = x.y;
    }
}

// grid (tokens, ranges).  part_o / part_ml as in attention_mixed_kernel (used when there are several ranges).
__global__ void __launch_bounds__(kThreads)
attention_mixed_decode_kernel(bf16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
                              const bf16* __restrict__ q, int64_t q_stride, const bf16* __restrict__ kcache,
                              const bf16* __restrict__ vcache, const float* __restrict__ mix, const float* __restrict__ sinks,
                              const int* __restrict__ start_pos, const int* __restrict__ block_table, int max_blocks,
                              DecShape sh, int page_size, int window, float scale) {
    extern __shared__ __align__(16) unsigned char smraw[];
    const int H = sh.H, G = sh.G, dk = sh.dk, dv = sh.dv, TK = sh.TK;
    const int per = H / G;
    const DecLayout L = dec_layout(sh);
    const int KP = G * dk + 8, VP = G * dv + 8, RP = TK + 1, PP = TK + 4;
    long long* where = reinterpret_cast<long long*>(smraw + L.where);
    float* qs = reinterpret_cast<float*>(smraw + L.q);          // [H * dk], scaled
    float* ms = reinterpret_cast<float*>(smraw + L.mix);        // [blocks of four heads][H][4]
    bf16* Ks = reinterpret_cast<bf16*>(smraw + L.k);            // [TK][KP]
    bf16* Vs = reinterpret_cast<bf16*>(smraw + L.v);            // [TK][VP]
    float* raw = reinterpret_cast<float*>(smraw + L.raw);       // [H][RP]
    float* pr = reinterpret_cast<float*>(smraw + L.p);          // [H][PP]: mixed scores, then weights
    float* mx = reinterpret_cast<float*>(smraw + L.stats);
    float* dn = mx + H;
    float* cr = dn + H;
    float* acc = reinterpret_cast<float*>(smraw + L.acc);       // [H * dv]
    const int tid = threadIdx.x;
    const int hb4 = (H + 3) / 4;
    for (int i = tid; i < hb4 * H * 4; i += kThreads) {
        const int u = i & 3, g = (i >> 2) % H, h = (i >> 2) / H * 4 + u;
        ms[i] = h < H ? mix[(size_t)h * H + g] : 0.f;
    }
    griddep_wait();
    griddep_launch();
    const int t = blockIdx.x;                                   // token t is request t
    const int pq = start_pos[t];
    int hi = pq, lo = window > 0 ? max(0, pq - window + 1) : 0;
    const int splits = gridDim.y, split = blockIdx.y;
    if (splits > 1) {
        const int chunk = (((hi - lo + 1) + splits - 1) / splits + TK - 1) / TK * TK;
        lo += split * chunk;
        hi = min(hi, lo + chunk - 1);
    }
    const int* table = block_table + (int64_t)t * max_blocks;
    for (int i = tid; i < H * dk; i += kThreads) qs[i] = __bfloat162float(q[(int64_t)t * q_stride + i]) * scale;
    for (int h = tid; h < H; h += kThreads) {
        mx[h] = (sinks && split == 0) ? sinks[h] : -INFINITY;
        dn[h] = (sinks && split == 0) ? 1.f : 0.f;
    }
    for (int i = tid; i < H * dv; i += kThreads) acc[i] = 0.f;
    const int k8 = G * dk / 8, v8 = G * dv / 8, dk8 = dk / 8, dv8 = dv / 8;

    for (int j0 = lo; j0 <= hi; j0 += TK) {
        const int nk = min(TK, hi - j0 + 1);
        __syncthreads();
        locate_keys(where, table, j0, nk, TK, G, page_size);
        __syncthreads();
        // keys and values of the tile, both on their way before either is used
#pragma unroll 4
        for (int i = tid; i < nk * k8; i += kThreads) {
            const int jj = i / k8, c = i - jj * k8, g = c / dk8, d = (c - g * dk8) * 8;
            const long long at = where[jj];
            uint4 v = make_uint4(0, 0, 0, 0);
            if (at >= 0) v = *reinterpret_cast<const uint4*>(kcache + (at + (long long)g * page_size) * dk + d);
            *reinterpret_cast<uint4*>(Ks + (size_t)jj * KP + g * dk + d) = v;
        }
#pragma unroll 4
        for (int i = tid; i < nk * v8; i += kThreads) {
            const int jj = i / v8, c = i - jj * v8, g = c / dv8, d = (c - g * dv8) * 8;
            const long long at = where[jj];
            uint4 v = make_uint4(0, 0, 0, 0);
            if (at >= 0) v = *reinterpret_cast<const uint4*>(vcache + (at + (long long)g * page_size) * dv + d);
            *reinterpret_cast<uint4*>(Vs + (size_t)jj * VP + g * dv + d) = v;
        }
        __syncthreads();
        // raw scores: a thread takes one key of one kv head and up to four of that kv head's query heads at a time
        const int ub = (per + 3) / 4;
        for (int it = tid; it < G * ub * TK; it += kThreads) {
            const int jj = it % TK, rest = it / TK, u0 = (rest % ub) * 4, g = rest / ub;
            if (jj >= nk) continue;
            const int nu = min(4, per - u0);
            const bf16* kr = Ks + (size_t)jj * KP + g * dk;
            const float* q0 = qs + (size_t)(g * per + u0) * dk;
            const float* q1 = q0 + (nu > 1 ? dk : 0);
            const float* q2 = q0 + (nu > 2 ? 2 * dk : 0);
            const float* q3 = q0 + (nu > 3 ? 3 * dk : 0);
            float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
            for (int d = 0; d < dk; d += 8) {
                float kf[8];
                widen8(*reinterpret_cast<const uint4*>(kr + d), kf);
#pragma unroll
                for (int e = 0; e < 8; e += 4) {
                    const float4 x0 = *reinterpret_cast<const float4*>(q0 + d + e), x1 = *reinterpret_cast<const float4*>(q1 + d + e);
                    const float4 x2 = *reinterpret_cast<const float4*>(q2 + d + e), x3 = *reinterpret_cast<const float4*>(q3 + d + e);
                    a0 = fmaf(x0.x, kf[e], a0); a0 = fmaf(x0.y, kf[e + 1], a0); a0 = fmaf(x0.z, kf[e + 2], a0); a0 = fmaf(x0.w, kf[e + 3], a0);
                    a1 = fmaf(x1.x, kf[e], a1); a1 = fmaf(x1.y, kf[e + 1], a1); a1 = fmaf(x1.z, kf[e + 2], a1); a1 = fmaf(x1.w, kf[e + 3], a1);
                    a2 = fmaf(x2.x, kf[e], a2); a2 = fmaf(x2.y, kf[e + 1], a2); a2 = fmaf(x2.z, kf[e + 2], a2); a2 = fmaf(x2.w, kf[e + 3], a2);
                    a3 = fmaf(x3.x, kf[e], a3); a3 = fmaf(x3.y, kf[e + 1], a3); a3 = fmaf(x3.z, kf[e + 2], a3); a3 = fmaf(x3.w, kf[e + 3], a3);
                }
            }
            float* rg = raw + (size_t)(g * per + u0) * RP + jj;
            rg[0] = a0;
            if (nu > 1) rg[RP] = a1;
            if (nu > 2) rg[2 * RP] = a2;
            if (nu > 3) rg[3 * RP] = a3;
        }
        __syncthreads();
        // mixing and mask: a thread takes one key for four heads
        for (int it = tid; it < hb4 * TK; it += kThreads) {
            const int jj = it % TK, b4 = it / TK, b0 = b4 * 4;
            const int pos = j0 + jj;
            const bool visible = jj < nk && pos <= pq && (window <= 0 || pq - pos < window);
            float a0 = -INFINITY, a1 = -INFINITY, a2 = -INFINITY, a3 = -INFINITY;
            if (visible) {
                a0 = a1 = a2 = a3 = 0.f;
                const float4* mw = reinterpret_cast<const float4*>(ms) + (size_t)b4 * H;
#pragma unroll 4
                for (int g = 0; g < H; g++) {
                    const float x = raw[(size_t)g * RP + jj];
                    const float4 m = mw[g];
                    a0 = fmaf(m.x, x, a0);
                    a1 = fmaf(m.y, x, a1);
                    a2 = fmaf(m.z, x, a2);
                    a3 = fmaf(m.w, x, a3);
                }
            }
            pr[(size_t)b0 * PP + jj] = a0;
            if (b0 + 1 < H) pr[(size_t)(b0 + 1) * PP + jj] = a1;
            if (b0 + 2 < H) pr[(size_t)(b0 + 2) * PP + jj] = a2;
            if (b0 + 3 < H) pr[(size_t)(b0 + 3) * PP + jj] = a3;
        }
        __syncthreads();
        // one warp per head: maximum, weights, denominator (TK <= 32: a lane per key)
        {
            const int lane = tid & 31, warp = tid >> 5;
            for (int h = warp; h < H; h += kThreads / 32) {
                float* row = pr + (size_t)h * PP;
                const float sc = lane < TK ? row[lane] : -INFINITY;
                const float m_old = mx[h];
                const float m_new = fmaxf(m_old, warp_max(sc));
                const float w = (sc == -INFINITY) ? 0.f : expf(sc - m_new);
                const float c = (m_old == -INFINITY) ? 0.f : expf(m_old - m_new);
                const float sum = warp_sum(w);
                if (lane < TK) row[lane] = w;
                if (lane == 0) {
                    mx[h] = m_new;
                    dn[h] = dn[h] * c + sum;
                    cr[h] = c;
                }
            }
        }
        __syncthreads();
        // output: a thread takes eight value channels of one head
        for (int it = tid; it < H * dv8; it += kThreads) {
            const int h = it / dv8, e = (it - h * dv8) * 8;
            const bf16* vr = Vs + (size_t)(h / per) * dv + e;
            const float* pw = pr + (size_t)h * PP;
            float a[8];
#pragma unroll
            for (int u = 0; u < 8; u++) a[u] = 0.f;
            for (int jj = 0; jj < nk; jj++) {
                float vf[8];
                widen8(*reinterpret_cast<const uint4*>(vr + (size_t)jj * VP), vf);
                const float w = pw[jj];
#pragma unroll
                for (int u = 0; u < 8; u++) a[u] = fmaf(w, vf[u], a[u]);
            }
            const float c = cr[h];
            float* o = acc + (size_t)h * dv + e;
#pragma unroll
            for (int u = 0; u < 8; u++) o[u] = o[u] * c + a[u];
        }
    }
    __syncthreads();
    if (splits > 1) {
        float* po = part_o + ((size_t)t * splits + split) * H * dv;
        for (int i = tid; i < H * dv; i += kThreads) po[i] = acc[i];
        float* pm = part_ml + ((size_t)t * splits + split) * H * 2;
        for (int h = tid; h < H; h += kThreads) {
            pm[2 * h] = mx[h];
            pm[2 * h + 1] = dn[h];
        }
        return;
    }
    for (int i = tid; i < H * dv; i += kThreads) {
        const float d = dn[i / dv];
        out[(int64_t)t * H * dv + i] = __float2bfloat16_rn(d > 0.f ? acc[i] / d : 0.f);
    }
}

// The key tile of the single-token form for these sizes; 0: the form does not take them.
inline DecShape dec_shape(int H, int G, int dk, int dv) {
    DecShape s = {H, G, dk, dv, 0};
    if (dk % 8 || dv % 8) return s;
    for (int tk = 32; tk >= 8; tk /= 2) {
        s.TK = tk;
        if (dec_layout(s).total <= 200 * 1024) return s;
    }
    s.TK = 0;
    return s;
}

// ---- the tensor-core form (bfloat16 portions) ---------------------------------------------------------
// The same sums with the two products on the tensor cores (mma.sync m16n8k16, bfloat16 operands, float32
// accumulators): a CTA takes a tile of 16 query rows and a block of HB output heads.  Per key tile it forms the raw
// scores of ALL heads (every output head needs them all), mixes them for its own heads in float32 on the CUDA
// cores, and keeps the output of its own heads in registers: 16 x HB x dv float32 values spread over the sixteen
// warps as m16n8 accumulator tiles.  The weights stay float32 until they meet the values: they enter the second
// product as two bfloat16 terms (the weight rounded, and what the rounding left), which keeps 16 bits of mantissa.
// Shared memory: the Q tile of all heads, the K tile of all kv heads (its place is reused for the transposed V tile
// of the block's own kv heads), the raw scores (their place is reused for the two-term weights), the mixed scores.
constexpr int kTile = 16;       // query rows of a tile
constexpr int kMmaThreads = 512; // sixteen warps: four a scheduler, so that one warp's waits are another's work
constexpr int kFrags = 8;       // m16n8 accumulator tiles a warp may own: HB * dv / 8 <= 16 * kFrags

struct MmaShape {
    int H, G, dk, dv, HB, TK;
};

__host__ __device__ inline int own_kv_heads(const MmaShape& s) {
    const int per = s.H / s.G;
    return (s.HB + per - 1) / per + 1;          // a block of HB heads touches at most this many kv heads
}

struct MmaLayout {
    size_t q, k, raw, mixed, stats, mix, where, total;
};

__host__ __device__ inline MmaLayout mma_layout(const MmaShape& s) {
    MmaLayout L;
    size_t o = 0;
    L.q = o;      o += (size_t)kTile * (s.H * s.dk + 8) * 2;
    const size_t ktile = (size_t)s.TK * (s.G * s.dk + 8) * 2;
    const size_t vtile = (size_t)own_kv_heads(s) * s.dv * (s.TK + 8) * 2;
    L.k = o;      o += (ktile > vtile ? ktile : vtile);
    const size_t raw = (size_t)s.H * kTile * (s.TK + 4) * 4;
    const size_t pw = 2 * (size_t)s.HB * kTile * (s.TK + 8) * 2;
    L.raw = o;    o += (raw > pw ? raw : pw);
    L.mixed = o;  o += (size_t)s.HB * kTile * (s.TK + 4) * 4;
    L.stats = o;  o += 3 * (size_t)s.HB * kTile * 4;
    L.mix = o;    o += ((size_t)s.HB * s.H * 4 + 15) / 16 * 16;
    L.where = o;  o += (size_t)s.TK * 8;
    L.total = (o + 15) / 16 * 16;
    return L;
}

__device__ __forceinline__ uint32_t ld32(const bf16* p) { return *reinterpret_cast<const uint32_t*>(p); }

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__global__ void __launch_bounds__(kMmaThreads)
attention_mixed_mma_kernel(bf16* __restrict__ out, const bf16* __restrict__ q, int64_t q_stride,
                           const bf16* __restrict__ kcache, const bf16* __restrict__ vcache,
                           const float* __restrict__ mix, const float* __restrict__ sinks,
                           const int* __restrict__ q_start, const int* __restrict__ start_pos,
                           const int* __restrict__ block_table, int max_blocks, int n_requests, MmaShape sh, int page_size,
                           int window, float scale) {
    extern __shared__ __align__(16) unsigned char smraw[];
    const int H = sh.H, G = sh.G, dk = sh.dk, dv = sh.dv, HB = sh.HB, TK = sh.TK;
    const int per = H / G;
    const MmaLayout L = mma_layout(sh);
    const int QP = H * dk + 8, KP = G * dk + 8, VP = TK + 8, RP = TK + 4, PP = TK + 8;
    bf16* Qs = reinterpret_cast<bf16*>(smraw + L.q);            // [16][QP]
    bf16* Ks = reinterpret_cast<bf16*>(smraw + L.k);            // [TK][KP]
    bf16* Vt = Ks;                                              // [own kv heads * dv][VP], after the scores
    float* raw = reinterpret_cast<float*>(smraw + L.raw);       // [H][16][RP]
    bf16* Ph = reinterpret_cast<bf16*>(smraw + L.raw);          // [HB][16][PP], after the mixing
    bf16* Pl = Ph + (size_t)HB * kTile * PP;
    float* mixed = reinterpret_cast<float*>(smraw + L.mixed);   // [HB][16][RP]
    float* mx = reinterpret_cast<float*>(smraw + L.stats);      // [HB][16]
    float* dn = mx + HB * kTile;
    float* cr = dn + HB * kTile;
    float* ms = reinterpret_cast<float*>(smraw + L.mix);        // [HB][H], times scale
    long long* where = reinterpret_cast<long long*>(smraw + L.where);   // [TK]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int fr = lane >> 2, fc = (lane & 3) * 2;              // a fragment's row and first column of this lane

    const int h0 = blockIdx.y * HB;
    const int nh = min(HB, H - h0);
    const int c_first = h0 / per;                               // first kv head of the block's own heads
    const int n_own = (h0 + nh - 1) / per - c_first + 1;
    for (int i = tid; i < nh * H; i += kMmaThreads) ms[i] = mix[(size_t)(h0 + i / H) * H + i % H] * scale;
    griddep_wait();
    griddep_launch();
    int req = 0, tile = blockIdx.x;
    for (; req < n_requests; req++) {
        const int tiles = (q_start[req + 1] - q_start[req] + kTile - 1) / kTile;
        if (tile < tiles) break;
        tile -= tiles;
    }
    if (req >= n_requests) return;
    const int row0 = q_start[req] + tile * kTile;
    const int nq = min(kTile, q_start[req + 1] - row0);
    const int p0 = start_pos[req] + tile * kTile;
    const int hi = p0 + nq - 1;
    const int lo = window > 0 ? max(0, p0 - window + 1) : 0;
    const int* table = block_table + (int64_t)req * max_blocks;

    // the Q tile of all heads, 16 bytes at a time; rows past the portion's end are zero
    const int qv = H * dk / 8;
    for (int i = tid; i < kTile * qv; i += kMmaThreads) {
        const int r = i / qv, c = i - r * qv;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < nq) v = *reinterpret_cast<const uint4*>(q + (int64_t)(row0 + r) * q_stride + c * 8);
        *reinterpret_cast<uint4*>(Qs + (size_t)r * QP + c * 8) = v;
    }
    for (int i = tid; i < HB * kTile; i += kMmaThreads) {
        const int h = h0 + i / kTile;
        mx[i] = (sinks && h < H) ? sinks[h] : -INFINITY;
        dn[i] = sinks ? 1.f : 0.f;
    }
    float acc[kFrags][4];
#pragma unroll
    for (int f = 0; f < kFrags; f++) acc[f][0] = acc[f][1] = acc[f][2] = acc[f][3] = 0.f;
    const int ntv = dv / 8;                     // accumulator tiles of a head
    const int n_tiles = nh * ntv;

    for (int j0 = lo; j0 <= hi; j0 += TK) {
        const int nk = min(TK, hi - j0 + 1);
        __syncthreads();                        // the tile before has been used up
        locate_keys(where, table, j0, nk, TK, G, page_size);
        __syncthreads();
        // (1) keys of all kv heads
        const int kv8 = dk / 8;
#pragma unroll 2
        for (int i = tid; i < TK * G * kv8; i += kMmaThreads) {
            const int jj = i / (G * kv8), rest = i - jj * (G * kv8), g = rest / kv8, c = rest - g * kv8;
            const long long at = where[jj];
            uint4 v = make_uint4(0, 0, 0, 0);
            if (at >= 0) v = *reinterpret_cast<const uint4*>(kcache + (at + (long long)g * page_size) * dk + c * 8);
            *reinterpret_cast<uint4*>(Ks + (size_t)jj * KP + g * dk + c * 8) = v;
        }
        __syncthreads();
        // (2) raw scores: a warp takes whole heads; A = the head's Q rows, B = its kv head's keys
        for (int g = warp; g < H; g += kMmaThreads / 32) {
            float c[4][4];
#pragma unroll
            for (int nt = 0; nt < 4; nt++) c[nt][0] = c[nt][1] = c[nt][2] = c[nt][3] = 0.f;
            const bf16* qa = Qs + (size_t)fr * QP + g * dk + fc;
            const bf16* kb = Ks + (size_t)fr * KP + (g / per) * dk + fc;
            for (int k0 = 0; k0 < dk; k0 += 16) {
                const uint32_t a0 = ld32(qa + k0), a1 = ld32(qa + 8 * QP + k0), a2 = ld32(qa + k0 + 8), a3 = ld32(qa + 8 * QP + k0 + 8);
#pragma unroll
                for (int nt = 0; nt < 4; nt++)
                    if (nt * 8 < TK) mma_bf16(c[nt], a0, a1, a2, a3, ld32(kb + (size_t)nt * 8 * KP + k0), ld32(kb + (size_t)nt * 8 * KP + k0 + 8));
            }
            float* rg = raw + (size_t)g * kTile * RP;
#pragma unroll
            for (int nt = 0; nt < 4; nt++)
                if (nt * 8 < TK) {
                    rg[fr * RP + nt * 8 + fc] = c[nt][0];
                    rg[fr * RP + nt * 8 + fc + 1] = c[nt][1];
                    rg[(fr + 8) * RP + nt * 8 + fc] = c[nt][2];
                    rg[(fr + 8) * RP + nt * 8 + fc + 1] = c[nt][3];
                }
        }
        __syncthreads();
        // (3) the values of the block's own kv heads, transposed, over the keys' place; the mixing and the mask
        // (a thread takes eight channels of one key: neighbouring threads take neighbouring keys, so that the
        // transposed stores of a warp fall into different banks)
        const int dv8 = dv / 8;
#pragma unroll 2
        for (int i = tid; i < TK * n_own * dv8; i += kMmaThreads) {
            const int jj = i % TK, rest = i / TK, e8 = rest % dv8, c = rest / dv8;
            const long long at = where[jj];
            uint4 v = make_uint4(0, 0, 0, 0);
            if (at >= 0) v = *reinterpret_cast<const uint4*>(vcache + (at + (long long)(c_first + c) * page_size) * dv + e8 * 8);
            const bf16* h = reinterpret_cast<const bf16*>(&v);
            bf16* o = Vt + (size_t)(c * dv + e8 * 8) * VP + jj;
#pragma unroll
            for (int u = 0; u < 8; u++) o[(size_t)u * VP] = h[u];
        }
        const int hb4 = (nh + 3) / 4;
        for (int it = tid; it < hb4 * kTile * TK; it += kMmaThreads) {
            const int jj = it % TK, i = (it / TK) % kTile, b0 = (it / (TK * kTile)) * 4;
            const int pos = j0 + jj, pi = p0 + i;
            const bool visible = jj < nk && i < nq && pos <= pi && (window <= 0 || pi - pos < window);
            float a0 = -INFINITY, a1 = -INFINITY, a2 = -INFINITY, a3 = -INFINITY;
            if (visible) {
                const float* m0 = ms + (size_t)b0 * H;
                const float* m1 = b0 + 1 < nh ? m0 + H : m0;
                const float* m2 = b0 + 2 < nh ? m0 + 2 * H : m0;
                const float* m3 = b0 + 3 < nh ? m0 + 3 * H : m0;
                a0 = a1 = a2 = a3 = 0.f;
                const float* rr = raw + (size_t)i * RP + jj;
                for (int g = 0; g < H; g++) {
                    const float r = rr[(size_t)g * kTile * RP];
                    a0 = fmaf(m0[g], r, a0);
                    a1 = fmaf(m1[g], r, a1);
                    a2 = fmaf(m2[g], r, a2);
                    a3 = fmaf(m3[g], r, a3);
                }
            }
            mixed[((b0 + 0) * kTile + i) * RP + jj] = a0;
            if (b0 + 1 < nh) mixed[((b0 + 1) * kTile + i) * RP + jj] = a1;
            if (b0 + 2 < nh) mixed[((b0 + 2) * kTile + i) * RP + jj] = a2;
            if (b0 + 3 < nh) mixed[((b0 + 3) * kTile + i) * RP + jj] = a3;
        }
        __syncthreads();
        // (4) one warp per (head, row): maximum, two-term weights, denominator
        // (a warp takes 32 / TK rows at a time, TK lanes each: TK is 16 or 32 and the rows' count is a multiple of 16)
        const int rpw = 32 / TK, sub = lane / TK, jl = lane - sub * TK;
        for (int r0 = warp * rpw; r0 < nh * kTile; r0 += (kMmaThreads / 32) * rpw) {
            const int rw = r0 + sub;
            const float s = mixed[(size_t)rw * RP + jl];
            const float m_old = mx[rw];
            float top = s;
            for (int o = TK >> 1; o > 0; o >>= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, o));
            const float m_new = fmaxf(m_old, top);
            const float w = (s == -INFINITY) ? 0.f : expf(s - m_new);
            const float c = (m_old == -INFINITY) ? 0.f : expf(m_old - m_new);
            float sum = w;
            for (int o = TK >> 1; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            const bf16 wh = __float2bfloat16_rn(w);
            Ph[(size_t)rw * PP + jl] = wh;
            Pl[(size_t)rw * PP + jl] = __float2bfloat16_rn(w - __bfloat162float(wh));
            if (jl == 0) {
                mx[rw] = m_new;
                dn[rw] = dn[rw] * c + sum;
                cr[rw] = c;
            }
        }
        __syncthreads();
        // (5) the output tiles this warp owns: tile t = (head of the block, eight value channels)
#pragma unroll
        for (int f = 0; f < kFrags; f++) {
            const int t = warp + f * (kMmaThreads / 32);
            if (t < n_tiles) {
                const int hb = t / ntv, nt = t - hb * ntv;
                const float c_lo = cr[hb * kTile + fr], c_hi = cr[hb * kTile + fr + 8];
                acc[f][0] *= c_lo; acc[f][1] *= c_lo; acc[f][2] *= c_hi; acc[f][3] *= c_hi;
                const bf16* pa = Ph + (size_t)(hb * kTile + fr) * PP + fc;
                const bf16* pb = Pl + (size_t)(hb * kTile + fr) * PP + fc;
                const bf16* vb = Vt + (size_t)(((h0 + hb) / per - c_first) * dv + nt * 8 + fr) * VP + fc;
                for (int k0 = 0; k0 < TK; k0 += 16) {
                    const uint32_t b0 = ld32(vb + k0), b1 = ld32(vb + k0 + 8);
                    mma_bf16(acc[f], ld32(pa + k0), ld32(pa + 8 * PP + k0), ld32(pa + k0 + 8), ld32(pa + 8 * PP + k0 + 8), b0, b1);
                    mma_bf16(acc[f], ld32(pb + k0), ld32(pb + 8 * PP + k0), ld32(pb + k0 + 8), ld32(pb + 8 * PP + k0 + 8), b0, b1);
                }
            }
        }
    }
    __syncthreads();
#pragma unroll
    for (int f = 0; f < kFrags; f++) {
        const int t = warp + f * (kMmaThreads / 32);
        if (t < n_tiles) {
            const int hb = t / ntv, nt = t - hb * ntv;
            const int col = (h0 + hb) * dv + nt * 8 + fc;
            const float d_lo = dn[hb * kTile + fr], d_hi = dn[hb * kTile + fr + 8];
            if (fr < nq) {
                const float inv = d_lo > 0.f ? 1.f / d_lo : 0.f;
                *reinterpret_cast<__nv_bfloat162*>(out + (int64_t)(row0 + fr) * H * dv + col) =
                    __floats2bfloat162_rn(acc[f][0] * inv, acc[f][1] * inv);
            }
            if (fr + 8 < nq) {
                const float inv = d_hi > 0.f ? 1.f / d_hi : 0.f;
                *reinterpret_cast<__nv_bfloat162*>(out + (int64_t)(row0 + fr + 8) * H * dv + col) =
                    __floats2bfloat162_rn(acc[f][2] * inv, acc[f][3] * inv);
            }
        }
    }
}

// ---- the tensor-core form over a thread-block cluster ------------------------------------------------------
// The CTAs that share a tile of 16 query rows form a cluster, one CTA per block of HB heads (H = NB * HB, NB <= 8).
// A CTA computes the raw scores of ITS heads only, against the keys of its own kv heads, and leaves them in its shared
// memory; after a cluster barrier every CTA mixes the scores of all heads for its own heads, reading the other
// blocks' raw scores from their shared memory (distributed shared memory), and goes on alone: softmax, weights in
// two bfloat16 terms, second product with the values of its own kv heads.  No score is computed twice, no CTA holds
// more than its own heads' queries, keys and values, and several CTAs fit an SM.  Two cluster barriers per key tile:
// before the raw scores are overwritten (all blocks have mixed the tile before) and after they are written.
constexpr int kClThreads = 256;
constexpr int kClFrags = 8;     // m16n8 accumulator tiles a warp may own: HB * dv / 8 <= 8 * kClFrags
constexpr int kClTK = 32;       // keys of a tile

struct ClShape {
    int H, G, dk, dv, HB, NB, KV;   // KV: the most kv heads a block's heads lie on
};

struct ClLayout {
    size_t q, k, raw, mixed, p, stats, mix, where, total;
};

__host__ __device__ inline ClLayout cl_layout(const ClShape& s) {
    ClLayout L;
    size_t o = 0;
    L.q = o;      o += (size_t)kTile * (s.HB * s.dk + 8) * 2;
    const size_t ktile = (size_t)kClTK * (s.KV * s.dk + 8) * 2;
    const size_t vtile = (size_t)s.KV * s.dv * (kClTK + 8) * 2;
    L.k = o;      o += (ktile > vtile ? ktile : vtile);
    L.raw = o;    o += (size_t)s.HB * kTile * (kClTK + 4) * 4;
    L.mixed = o;  o += (size_t)s.HB * kTile * (kClTK + 4) * 4;
    L.p = o;      o += 2 * (size_t)s.HB * kTile * (kClTK + 8) * 2;
    L.stats = o;  o += 3 * (size_t)s.HB * kTile * 4;
    L.mix = o;    o += (size_t)((s.HB + 3) / 4) * s.H * 4 * 4;        // [blocks of four heads][H][4]
    L.where = o;  o += (size_t)kClTK * 8;
    L.total = (o + 15) / 16 * 16;
    return L;
}

__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}

// The address, in this CTA's shared window, of `p` as it lies in the shared memory of the cluster's CTA `rank`.
__device__ __forceinline__ const float* peer_shared(const float* p, unsigned rank) {
    uint64_t out;
    asm volatile("mapa.u64 %0, %1, %2;\n" : "=l"(out) : "l"((uint64_t)p), "r"(rank));
    return reinterpret_cast<const float*>(out);
}

__global__ void __launch_bounds__(kClThreads, 3)
attention_mixed_cluster_kernel(bf16* __restrict__ out, const bf16* __restrict__ q, int64_t q_stride,
                               const bf16* __restrict__ kcache, const bf16* __restrict__ vcache,
                               const float* __restrict__ mix, const float* __restrict__ sinks,
                               const int* __restrict__ q_start, const int* __restrict__ start_pos,
                               const int* __restrict__ block_table, int max_blocks, int n_requests, ClShape sh,
                               int page_size, int window, float scale) {
    extern __shared__ __align__(16) unsigned char smraw[];
    const int H = sh.H, G = sh.G, dk = sh.dk, dv = sh.dv, HB = sh.HB, NB = sh.NB;
    constexpr int TK = kClTK;
    const int per = H / G;
    const ClLayout L = cl_layout(sh);
    const int QP = HB * dk + 8, KP = sh.KV * dk + 8, VP = TK + 8, RP = TK + 4, PP = TK + 8;
    bf16* Qs = reinterpret_cast<bf16*>(smraw + L.q);            // [16][QP]: the block's own heads
    bf16* Ks = reinterpret_cast<bf16*>(smraw + L.k);            // [TK][KP]: the block's own kv heads
    bf16* Vt = Ks;                                              // [own kv heads * dv][VP], after the scores
    float* raw = reinterpret_cast<float*>(smraw + L.raw);       // [HB][16][RP]: read by the whole cluster
    float* mixed = reinterpret_cast<float*>(smraw + L.mixed);   // [HB][16][RP]
    bf16* Ph = reinterpret_cast<bf16*>(smraw + L.p);            // [HB][16][PP]
    bf16* Pl = Ph + (size_t)HB * kTile * PP;
    float* mx = reinterpret_cast<float*>(smraw + L.stats);
    float* dn = mx + HB * kTile;
    float* cr = dn + HB * kTile;
    float* ms = reinterpret_cast<float*>(smraw + L.mix);        // [blocks of four own heads][H][4], times scale
    long long* where = reinterpret_cast<long long*>(smraw + L.where);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int fr = lane >> 2, fc = (lane & 3) * 2;

    const int rank = blockIdx.y;                                // the cluster spans the grid's y: the rank in it
    const int h0 = rank * HB;
    const int c_first = h0 / per;
    const int n_own = (h0 + HB - 1) / per - c_first + 1;
    for (int i = tid; i < ((HB + 3) / 4) * H * 4; i += kClThreads) {
        const int u = i & 3, g = (i >> 2) % H, hb = (i >> 2) / H * 4 + u;     // weight of head g in own head hb
        ms[i] = hb < HB ? mix[(size_t)(h0 + hb) * H + g] * scale : 0.f;
    }
    griddep_wait();
    griddep_launch();
    int req = 0, tile = blockIdx.x;
    for (; req < n_requests; req++) {
        const int tiles = (q_start[req + 1] - q_start[req] + kTile - 1) / kTile;
        if (tile < tiles) break;
        tile -= tiles;
    }
    if (req >= n_requests) return;                              // the same for every CTA of the cluster
    const int row0 = q_start[req] + tile * kTile;
    const int nq = min(kTile, q_start[req + 1] - row0);
    const int p0 = start_pos[req] + tile * kTile;
    const int hi = p0 + nq - 1;
    const int lo = window > 0 ? max(0, p0 - window + 1) : 0;
    const int* table = block_table + (int64_t)req * max_blocks;

    const int qv = HB * dk / 8;
    for (int i = tid; i < kTile * qv; i += kClThreads) {
        const int r = i / qv, c = i - r * qv;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < nq) v = *reinterpret_cast<const uint4*>(q + (int64_t)(row0 + r) * q_stride + (size_t)h0 * dk + c * 8);
        *reinterpret_cast<uint4*>(Qs + (size_t)r * QP + c * 8) = v;
    }
    for (int i = tid; i < HB * kTile; i += kClThreads) {
        mx[i] = sinks ? sinks[h0 + i / kTile] : -INFINITY;
        dn[i] = sinks ? 1.f : 0.f;
    }
    float acc[kClFrags][4];
#pragma unroll
    for (int f = 0; f < kClFrags; f++) acc[f][0] = acc[f][1] = acc[f][2] = acc[f][3] = 0.f;
    const int ntv = dv / 8;
    const int n_tiles = HB * ntv;
    const float* peer_raw[8];
#pragma unroll
    for (int r = 0; r < 8; r++) peer_raw[r] = peer_shared(raw, r < NB ? r : 0);

    for (int j0 = lo; j0 <= hi; j0 += TK) {
        const int nk = min(TK, hi - j0 + 1);
        cluster_sync_all();                     // every block has mixed the tile before: raw may be overwritten
        locate_keys(where, table, j0, nk, TK, G, page_size);
        __syncthreads();
        // (1) keys of the block's own kv heads
        const int kv8 = dk / 8;
#pragma unroll 2
        for (int i = tid; i < TK * n_own * kv8; i += kClThreads) {
            const int jj = i / (n_own * kv8), rest = i - jj * (n_own * kv8), c = rest / kv8, d8 = rest - c * kv8;
            const long long at = where[jj];
            uint4 v = make_uint4(0, 0, 0, 0);
            if (at >= 0) v = *reinterpret_cast<const uint4*>(kcache + (at + (long long)(c_first + c) * page_size) * dk + d8 * 8);
            *reinterpret_cast<uint4*>(Ks + (size_t)jj * KP + c * dk + d8 * 8) = v;
        }
        __syncthreads();
        // (2) raw scores of the block's own heads: a unit is (head, eight keys)
        for (int u = warp; u < HB * (TK / 8); u += kClThreads / 32) {
            const int hb = u / (TK / 8), nt = u - hb * (TK / 8);
            float c[4] = {0.f, 0.f, 0.f, 0.f};
            const bf16* qa = Qs + (size_t)fr * QP + hb * dk + fc;
            const bf16* kb = Ks + (size_t)(nt * 8 + fr) * KP + ((h0 + hb) / per - c_first) * dk + fc;
#pragma unroll 4
            for (int k0 = 0; k0 < dk; k0 += 16)
                mma_bf16(c, ld32(qa + k0), ld32(qa + 8 * QP + k0), ld32(qa + k0 + 8), ld32(qa + 8 * QP + k0 + 8), ld32(kb + k0),
                         ld32(kb + k0 + 8));
            float* rg = raw + (size_t)hb * kTile * RP + nt * 8 + fc;
            rg[fr * RP] = c[0];
            rg[fr * RP + 1] = c[1];
            rg[(fr + 8) * RP] = c[2];
            rg[(fr + 8) * RP + 1] = c[3];
        }
        cluster_sync_all();                     // the raw scores of all blocks are written
        // (3) the values of the block's own kv heads, transposed, over the keys' place; the mixing and the mask
        const int dv8 = dv / 8;
#pragma unroll 2
        for (int i = tid; i < TK * n_own * dv8; i += kClThreads) {
            const int jj = i % TK, rest = i / TK, e8 = rest % dv8, c = rest / dv8;
            const long long at = where[jj];
            uint4 v = make_uint4(0, 0, 0, 0);
            if (at >= 0) v = *reinterpret_cast<const uint4*>(vcache + (at + (long long)(c_first + c) * page_size) * dv + e8 * 8);
            const bf16* h = reinterpret_cast<const bf16*>(&v);
            bf16* o = Vt + (size_t)(c * dv + e8 * 8) * VP + jj;
#pragma unroll
            for (int u = 0; u < 8; u++) o[(size_t)u * VP] = h[u];
        }
        // (a thread mixes two neighbouring keys of one row for four own heads: one 8-byte read of a raw score pair and
        // one 16-byte read of the four heads' weights serve eight sums)
        const int hb4 = (HB + 3) / 4;
        for (int it = tid; it < hb4 * kTile * (TK / 2); it += kClThreads) {
            const int j2 = it % (TK / 2), i = (it / (TK / 2)) % kTile, b4 = it / ((TK / 2) * kTile);
            const int b0 = b4 * 4;
            float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f, c0 = 0.f, c1 = 0.f, c2 = 0.f, c3 = 0.f;
            if (i < nq) {
                const int off = i * RP + 2 * j2;
                const float4* mw = reinterpret_cast<const float4*>(ms) + (size_t)b4 * H;
#pragma unroll
                for (int r = 0; r < 8; r++) {
                    if (r < NB) {
                        const float* rr = peer_raw[r] + off;
#pragma unroll 4
                        for (int gg = 0; gg < HB; gg++) {
                            const float2 x = *reinterpret_cast<const float2*>(rr + (size_t)gg * kTile * RP);
                            const float4 m = mw[r * HB + gg];
                            a0 = fmaf(m.x, x.x, a0); c0 = fmaf(m.x, x.y, c0);
                            a1 = fmaf(m.y, x.x, a1); c1 = fmaf(m.y, x.y, c1);
                            a2 = fmaf(m.z, x.x, a2); c2 = fmaf(m.z, x.y, c2);
                            a3 = fmaf(m.w, x.x, a3); c3 = fmaf(m.w, x.y, c3);
                        }
                    }
                }
            }
            const int pi = p0 + i, pos = j0 + 2 * j2;
            const bool v0 = 2 * j2 < nk && i < nq && pos <= pi && (window <= 0 || pi - pos < window);
            const bool v1 = 2 * j2 + 1 < nk && i < nq && pos + 1 <= pi && (window <= 0 || pi - pos - 1 < window);
            float* dst = mixed + (size_t)(b0 * kTile + i) * RP + 2 * j2;
            *reinterpret_cast<float2*>(dst) = make_float2(v0 ? a0 : -INFINITY, v1 ? c0 : -INFINITY);
            if (b0 + 1 < HB) *reinterpret_cast<float2*>(dst + kTile * RP) = make_float2(v0 ? a1 : -INFINITY, v1 ? c1 : -INFINITY);
            if (b0 + 2 < HB) *reinterpret_cast<float2*>(dst + 2 * kTile * RP) = make_float2(v0 ? a2 : -INFINITY, v1 ? c2 : -INFINITY);
            if (b0 + 3 < HB) *reinterpret_cast<float2*>(dst + 3 * kTile * RP) = make_float2(v0 ? a3 : -INFINITY, v1 ? c3 : -INFINITY);
        }
        __syncthreads();
        // (4) four lanes per (head, row), eight keys each: maximum, two-term weights, denominator
        for (int r0 = warp * 8; r0 < HB * kTile; r0 += (kClThreads / 32) * 8) {
            const int rw = r0 + (lane >> 2), part = lane & 3;
            const float* src = mixed + (size_t)rw * RP + part * 8;
            const float m_old = mx[rw], d_old = dn[rw];
            float sc[8];
            float top = -INFINITY;
#pragma unroll
            for (int t = 0; t < 8; t++) {
                sc[t] = src[t];
                top = fmaxf(top, sc[t]);
            }
            top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, 1));
            top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, 2));
            const float m_new = fmaxf(m_old, top);
            float sum = 0.f;
            uint32_t* ph = reinterpret_cast<uint32_t*>(Ph + (size_t)rw * PP + part * 8);
            uint32_t* pl = reinterpret_cast<uint32_t*>(Pl + (size_t)rw * PP + part * 8);
#pragma unroll
            for (int t = 0; t < 8; t += 2) {
                const float w0 = (sc[t] == -INFINITY) ? 0.f : expf(sc[t] - m_new);
                const float w1 = (sc[t + 1] == -INFINITY) ? 0.f : expf(sc[t + 1] - m_new);
                sum += w0 + w1;
                const __nv_bfloat162 hi = __floats2bfloat162_rn(w0, w1);
                const float2 back = __bfloat1622float2(hi);
                const __nv_bfloat162 lo = __floats2bfloat162_rn(w0 - back.x, w1 - back.y);
                ph[t >> 1] = *reinterpret_cast<const uint32_t*>(&hi);
                pl[t >> 1] = *reinterpret_cast<const uint32_t*>(&lo);
            }
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            if (part == 0) {
                const float c = (m_old == -INFINITY) ? 0.f : expf(m_old - m_new);
                mx[rw] = m_new;
                dn[rw] = d_old * c + sum;
                cr[rw] = c;
            }
        }
        __syncthreads();
        // (5) the output tiles this warp owns
#pragma unroll
        for (int f = 0; f < kClFrags; f++) {
            const int t = warp + f * (kClThreads / 32);
            if (t < n_tiles) {
                const int hb = t / ntv, nt = t - hb * ntv;
                const float c_lo = cr[hb * kTile + fr], c_hi = cr[hb * kTile + fr + 8];
                acc[f][0] *= c_lo; acc[f][1] *= c_lo; acc[f][2] *= c_hi; acc[f][3] *= c_hi;
                const bf16* pa = Ph + (size_t)(hb * kTile + fr) * PP + fc;
                const bf16* pb = Pl + (size_t)(hb * kTile + fr) * PP + fc;
                const bf16* vb = Vt + (size_t)(((h0 + hb) / per - c_first) * dv + nt * 8 + fr) * VP + fc;
#pragma unroll
                for (int k0 = 0; k0 < TK; k0 += 16) {
                    const uint32_t b0 = ld32(vb + k0), b1 = ld32(vb + k0 + 8);
                    mma_bf16(acc[f], ld32(pa + k0), ld32(pa + 8 * PP + k0), ld32(pa + k0 + 8), ld32(pa + 8 * PP + k0 + 8), b0, b1);
                    mma_bf16(acc[f], ld32(pb + k0), ld32(pb + 8 * PP + k0), ld32(pb + k0 + 8), ld32(pb + 8 * PP + k0 + 8), b0, b1);
                }
            }
        }
    }
    cluster_sync_all();                         // no block leaves while another may still read its raw scores
#pragma unroll
    for (int f = 0; f < kClFrags; f++) {
        const int t = warp + f * (kClThreads / 32);
        if (t < n_tiles) {
            const int hb = t / ntv, nt = t - hb * ntv;
            const int col = (h0 + hb) * dv + nt * 8 + fc;
            const float d_lo = dn[hb * kTile + fr], d_hi = dn[hb * kTile + fr + 8];
            if (fr < nq) {
                const float inv = d_lo > 0.f ? 1.f / d_lo : 0.f;
                *reinterpret_cast<__nv_bfloat162*>(out + (int64_t)(row0 + fr) * H * dv + col) =
                    __floats2bfloat162_rn(acc[f][0] * inv, acc[f][1] * inv);
            }
            if (fr + 8 < nq) {
                const float inv = d_hi > 0.f ? 1.f / d_hi : 0.f;
                *reinterpret_cast<__nv_bfloat162*>(out + (int64_t)(row0 + fr + 8) * H * dv + col) =
                    __floats2bfloat162_rn(acc[f][2] * inv, acc[f][3] * inv);
            }
        }
    }
}

// The blocks of heads of the cluster form for these sizes; NB 0: the form does not take them.
inline ClShape cl_shape(int H, int G, int dk, int dv) {
    ClShape s = {H, G, dk, dv, 0, 0, 0};
    if (dk % 16 || dv % 16) return s;
    const int per = H / G;
    for (int nb = 8; nb >= 2; nb--) {
        if (H % nb) continue;
        const int hb = H / nb;
        if (hb * (dv / 8) > (kClThreads / 32) * kClFrags) continue;
        s.HB = hb;
        s.NB = nb;
        s.KV = hb % per == 0 ? hb / per : (per % hb == 0 ? 1 : (hb + per - 1) / per + 1);
        if (cl_layout(s).total <= 110 * 1024) return s;
    }
    s.NB = 0;
    return s;
}

// The block of heads and the key tile of the tensor-core form for these sizes; HB 0: the form does not take them.
inline MmaShape mma_shape(int H, int G, int dk, int dv) {
    MmaShape s = {H, G, dk, dv, 0, 0};
    if (dk % 16 || dv % 16 || dv > (kMmaThreads / 32) * kFrags * 8) return s;
    int hb = (kMmaThreads / 32) * kFrags * 8 / dv;
    if (hb > H) hb = H;
    for (int tk = 32; tk >= 16; tk /= 2) {
        s.HB = hb;
        s.TK = tk;
        if (mma_layout(s).total <= 220 * 1024) return s;
    }
    s.HB = 0;
    return s;
}

}  // namespace

// out [n][H * dv] contiguous and q [n][H * dk] (row stride q_stride) in the element type `dtype`, which is also
// the caches' ([pages][G][page_size][dk] and [pages][G][page_size][dv]); mix float32 [H][H]; sinks float32 [H]
// or NULL; request s brings rows q_start[s] .. q_start[s + 1] at positions start_pos[s] ...; tile_rows: rows of a
// query tile (1 for single tokens), n_tiles: an upper bound of the tiles (sum over requests of ceil(rows / tile_rows)).
// splits > 1 (tile_rows 1 and every request one token): the keys of a token are cut into that many ranges, one CTA each,
// their results left in part_o float32 [tokens][splits][H * dv] and part_ml float32 [tokens][splits][H][2] and joined by a
// second kernel.
extern "C" int kllm_attention_mixed(void* out, const void* q, int64_t q_stride, const void* kcache, const void* vcache,
                                    const float* mix, const float* sinks, const int* q_start, const int* start_pos,
                                    const int* block_table, int max_blocks, int n_requests, int n_tiles, int tile_rows,
                                    int n_heads, int n_kv, int dk, int dv, int page_size, int window, float scale,
                                    int splits, float* part_o, float* part_ml, int dtype, void* stream) {
    if (n_requests <= 0 || n_tiles <= 0) return 0;
    if (n_heads <= 0 || n_kv <= 0 || n_heads % n_kv || dk <= 0 || dv <= 0 || page_size <= 0)
        KLLM_FAIL("mixed attention: %d heads on %d kv heads of sizes %d, %d", n_heads, n_kv, dk, dv);
    if (tile_rows < 1 || tile_rows > kMaxTQ) KLLM_FAIL("mixed attention: tiles of %d rows (1 to %d)", tile_rows, kMaxTQ);
    if (splits < 1 || (splits > 1 && (tile_rows != 1 || n_tiles != n_requests || !part_o || !part_ml)))
        KLLM_FAIL("mixed attention: %d key ranges need single tokens and room for the ranges' results", splits);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == KLLM_BF16 && tile_rows == 1 && n_tiles == n_requests && dec_shape(n_heads, n_kv, dk, dv).TK > 0 &&
        !(((uintptr_t)kcache | (uintptr_t)vcache) & 15)) {
        // every request one token: the form that keeps the tiles in bfloat16 (token t is request t)
        const DecShape ds = dec_shape(n_heads, n_kv, dk, dv);
        const size_t need = dec_layout(ds).total;
        static bool raised_dec = false;
        if (need > 48 * 1024 && !raised_dec) {
            cudaFuncSetAttribute(attention_mixed_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
            raised_dec = true;
        }
        kllm_launch((attention_mixed_decode_kernel), dim3(n_tiles, splits), dim3(kThreads), need, s, (bf16*)out, part_o, part_ml,
                    (const bf16*)q, q_stride, (const bf16*)kcache, (const bf16*)vcache, mix, sinks, start_pos, block_table,
                    max_blocks, ds, page_size, window, scale);
        if (splits > 1) {
            cudaError_t e = cudaGetLastError();
            if (e != cudaSuccess) KLLM_FAIL("mixed attention: %s", cudaGetErrorString(e));
            kllm_launch((attention_mixed_merge_kernel<bf16>), dim3(n_tiles, n_heads), dim3(128), 0, s, (bf16*)out, part_o, part_ml,
                        splits, n_heads, dv);
        }
        KLLM_LAUNCH_STATUS();
    }
    const size_t budget = 200 * 1024;
    Shape sh = {n_heads, n_kv, dk, dv, tile_rows, 32};
    while (sh.TK > 4 && smem_floats(sh) * sizeof(float) > budget) sh.TK /= 2;
    while (sh.TQ > 1 && smem_floats(sh) * sizeof(float) > budget) sh.TQ /= 2;
    if (sh.TQ != tile_rows) KLLM_FAIL("mixed attention: tiles of %d rows do not fit shared memory (%d would)", tile_rows, sh.TQ);
    const size_t smem = smem_floats(sh) * sizeof(float);
    if (smem > budget) KLLM_FAIL("mixed attention: %d heads of sizes %d, %d do not fit shared memory", n_heads, dk, dv);
    static bool raised[2] = {false, false};
    if (dtype == KLLM_F32) {
        if (smem > 48 * 1024 && !raised[0]) {
            cudaFuncSetAttribute(attention_mixed_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)budget);
            raised[0] = true;
        }
        kllm_launch((attention_mixed_kernel<float>), dim3(n_tiles, splits), dim3(kThreads), smem, s, (float*)out, part_o, part_ml, (const float*)q,
                    q_stride, (const float*)kcache, (const float*)vcache, mix, sinks, q_start, start_pos, block_table,
                    max_blocks, n_requests, sh, page_size, window, scale);
    } else if (dtype == KLLM_BF16) {
        if (smem > 48 * 1024 && !raised[1]) {
            cudaFuncSetAttribute(attention_mixed_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)budget);
            raised[1] = true;
        }
        kllm_launch((attention_mixed_kernel<bf16>), dim3(n_tiles, splits), dim3(kThreads), smem, s, (bf16*)out, part_o, part_ml, (const bf16*)q,
                    q_stride, (const bf16*)kcache, (const bf16*)vcache, mix, sinks, q_start, start_pos, block_table,
                    max_blocks, n_requests, sh, page_size, window, scale);
    } else {
        KLLM_FAIL("mixed attention: unknown element type %d", dtype);
    }
    if (splits > 1) {
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) KLLM_FAIL("mixed attention: %s", cudaGetErrorString(e));
        if (dtype == KLLM_F32)
            kllm_launch((attention_mixed_merge_kernel<float>), dim3(n_tiles, n_heads), dim3(128), 0, s, (float*)out, part_o, part_ml,
                        splits, n_heads, dv);
        else
            kllm_launch((attention_mixed_merge_kernel<bf16>), dim3(n_tiles, n_heads), dim3(128), 0, s, (bf16*)out, part_o, part_ml,
                        splits, n_heads, dv);
    }
    KLLM_LAUNCH_STATUS();
}

// The keys of a tile on the CUDA-core form for these sizes and rows (what the cutting into ranges counts in).
extern "C" int kllm_attention_mixed_tile_keys(int n_heads, int n_kv, int dk, int dv, int tile_rows) {
    // (the bfloat16 single-token form's tile where it takes the sizes: the float32 form's tiles are no larger, and
    // every form cuts the ranges in whole tiles of its own)
    if (tile_rows == 1 && dec_shape(n_heads, n_kv, dk, dv).TK > 0) return dec_shape(n_heads, n_kv, dk, dv).TK;
    Shape sh = {n_heads, n_kv, dk, dv, tile_rows, 32};
    while (sh.TK > 4 && smem_floats(sh) * sizeof(float) > 200 * 1024) sh.TK /= 2;
    return sh.TK;
}

// The most rows a query tile of these sizes may have, at most 8: what fits shared memory beside a tile of 16
// keys, or one row beside a smaller key tile; 0 when not even that fits.
extern "C" int kllm_attention_mixed_tile_rows(int n_heads, int n_kv, int dk, int dv) {
    if (n_heads <= 0 || n_kv <= 0 || dk <= 0 || dv <= 0) return 0;
    Shape sh = {n_heads, n_kv, dk, dv, kMaxTQ, 16};
    while (sh.TQ > 1 && smem_floats(sh) * sizeof(float) > 200 * 1024) sh.TQ /= 2;
    while (sh.TK > 4 && smem_floats(sh) * sizeof(float) > 200 * 1024) sh.TK /= 2;
    return smem_floats(sh) * sizeof(float) > 200 * 1024 ? 0 : sh.TQ;
}

// Whether the tensor-core form takes these sizes (bfloat16; head sizes in steps of 16; shared memory).
extern "C" int kllm_attention_mixed_mma_fits(int n_heads, int n_kv, int dk, int dv) {
    if (n_heads <= 0 || n_kv <= 0 || n_heads % n_kv || dk <= 0 || dv <= 0) return 0;
    return mma_shape(n_heads, n_kv, dk, dv).HB > 0 ? 1 : 0;
}

// The tensor-core form for bfloat16 portions: operands as in kllm_attention_mixed; n_tiles: an upper bound of the tiles of
// 16 rows (sum over requests of ceil(rows / 16)); q rows and the caches' rows 16-byte aligned.
extern "C" int kllm_attention_mixed_mma(void* out, const void* q, int64_t q_stride, const void* kcache, const void* vcache,
                                        const float* mix, const float* sinks, const int* q_start, const int* start_pos,
                                        const int* block_table, int max_blocks, int n_requests, int n_tiles, int n_heads,
                                        int n_kv, int dk, int dv, int page_size, int window, float scale, void* stream) {
    if (n_requests <= 0 || n_tiles <= 0) return 0;
    if (n_heads <= 0 || n_kv <= 0 || n_heads % n_kv || page_size <= 0)
        KLLM_FAIL("mixed attention: %d heads on %d kv heads", n_heads, n_kv);
    const MmaShape sh = mma_shape(n_heads, n_kv, dk, dv);
    if (sh.HB <= 0) KLLM_FAIL("mixed attention (tensor cores): head sizes %d, %d of %d heads are not taken", dk, dv, n_heads);
    if (((uintptr_t)q & 15) || (q_stride % 8) || ((uintptr_t)kcache & 15) || ((uintptr_t)out & 3))
        KLLM_FAIL("mixed attention (tensor cores): rows must be 16-byte aligned");
    const size_t smem = mma_layout(sh).total;
    static bool raised = false;
    if (smem > 48 * 1024 && !raised) {
        cudaError_t e = cudaFuncSetAttribute(attention_mixed_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
        if (e != cudaSuccess) KLLM_FAIL("mixed attention (tensor cores): %s", cudaGetErrorString(e));
        raised = true;
    }
    const int groups = (n_heads + sh.HB - 1) / sh.HB;
    kllm_launch((attention_mixed_mma_kernel), dim3(n_tiles, groups), dim3(kMmaThreads), smem, (cudaStream_t)stream, (bf16*)out,
                (const bf16*)q, q_stride, (const bf16*)kcache, (const bf16*)vcache, mix, sinks, q_start, start_pos, block_table,
                max_blocks, n_requests, sh, page_size, window, scale);
    KLLM_LAUNCH_STATUS();
}

// Whether the cluster form takes these sizes (bfloat16; head sizes in steps of 16; the heads in 2 to 8 equal blocks).
extern "C" int kllm_attention_mixed_cluster_fits(int n_heads, int n_kv, int dk, int dv) {
    if (n_heads <= 0 || n_kv <= 0 || n_heads % n_kv || dk <= 0 || dv <= 0) return 0;
    return cl_shape(n_heads, n_kv, dk, dv).NB > 0 ? 1 : 0;
}

// The cluster form for bfloat16 portions: operands as in kllm_attention_mixed_mma.  Returns -3 when the device cannot
// place a cluster of these CTAs, for the caller to take another form.
extern "C" int kllm_attention_mixed_cluster(void* out, const void* q, int64_t q_stride, const void* kcache, const void* vcache,
                                            const float* mix, const float* sinks, const int* q_start, const int* start_pos,
                                            const int* block_table, int max_blocks, int n_requests, int n_tiles, int n_heads,
                                            int n_kv, int dk, int dv, int page_size, int window, float scale, void* stream) {
    if (n_requests <= 0 || n_tiles <= 0) return 0;
    if (n_heads <= 0 || n_kv <= 0 || n_heads % n_kv || page_size <= 0)
        KLLM_FAIL("mixed attention: %d heads on %d kv heads", n_heads, n_kv);
    const ClShape sh = cl_shape(n_heads, n_kv, dk, dv);
    if (sh.NB <= 0) KLLM_FAIL("mixed attention (cluster): head sizes %d, %d of %d heads are not taken", dk, dv, n_heads);
    if (((uintptr_t)q & 15) || (q_stride % 8) || ((uintptr_t)kcache & 15) || ((uintptr_t)vcache & 15) || ((uintptr_t)out & 3))
        KLLM_FAIL("mixed attention (cluster): rows must be 16-byte aligned");
    const size_t smem = cl_layout(sh).total;
    static bool raised = false;
    if (!raised) {
        cudaError_t e = cudaFuncSetAttribute(attention_mixed_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 110 * 1024);
        if (e != cudaSuccess) KLLM_FAIL("mixed attention (cluster): %s", cudaGetErrorString(e));
        raised = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_tiles, sh.NB);
    cfg.blockDim = dim3(kClThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = sh.NB;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    static int placeable[9] = {-1, -1, -1, -1, -1, -1, -1, -1, -1};
    if (placeable[sh.NB] < 0) {
        int clusters = 0;
        cudaError_t e = cudaOccupancyMaxActiveClusters(&clusters, attention_mixed_cluster_kernel, &cfg);
        placeable[sh.NB] = (e == cudaSuccess && clusters > 0) ? 1 : 0;
        if (e != cudaSuccess) cudaGetLastError();
    }
    if (!placeable[sh.NB]) return -3;
    cudaError_t e = cudaLaunchKernelEx(&cfg, attention_mixed_cluster_kernel, (bf16*)out, (const bf16*)q, q_stride,
                                       (const bf16*)kcache, (const bf16*)vcache, mix, sinks, q_start, start_pos, block_table,
                                       max_blocks, n_requests, sh, page_size, window, scale);
    if (e != cudaSuccess) KLLM_FAIL("mixed attention (cluster): %s", cudaGetErrorString(e));
    KLLM_LAUNCH_STATUS();
}
