// Grouped-query softmax attention whose softmax weights are mixed across the heads AFTER the softmax,
//   w_g[i][j] = softmax_j( scale * q_g[i] . k[j] + bias[min(i - j, far)][g] ),   w'_h = sum_g talk[h][g] w_g,
//   o_h[i] = sigmoid(gate[i][h]) * sum_j w'_h[i][j] v[j],
// over a causal mask that may be cut into chunks counted from position 0.  Mixing normalised weights needs every head's
// softmax denominator before any value is read, so the work is two passes over the keys:
//   stats  one CTA per (query tile, key/value group, key share): maximum and sum of exponentials of every (query, head);
//   apply  one CTA per (query tile, key share): recomputes the scores of ALL heads for a key tile, turns them into
//          normalised weights, mixes them across the heads in shared memory and multiplies with the values.
// Because the weights are normalised with the final statistics, the key shares' partial results simply add (merge kernel,
// fixed order).  Scores, weights and sums are fp32; keys and values come from the paged cache in its element type.
// Without mixing (talk == nullptr) the same two passes run with one key/value group per CTA.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>

#include <algorithm>

#include "asd_internal.h"
#include "blocks.h"
#include "elem.cuh"
#include "mixed_attention.h"

namespace asd {

namespace {

constexpr int KT = 64;          // keys per tile
constexpr int PS = KT + 16;     // floats between the weight rows of a tile (two rows of a warp fall into different banks)
constexpr int NT = 256;         // threads: 16 row lanes (ty) x 16 key / column lanes (tx)
constexpr int MAX_ROWS = 128;   // (head, query) pairs of a CTA
constexpr int SLOTS = 8;        // result rows a thread accumulates (over all of the CTA's key/value groups)


struct Layout {
    int q, kv, p, w, talk, m, l, off, total;   // float offsets
};
__host__ __device__ inline Layout mix_layout(int rows, int dkp, int dvp, int heads, bool apply, bool talk) {
    Layout L;
    int o = 0;
    L.q = o, o += rows * dkp;
    const int kvw = (dkp + 4) > dvp ? (dkp + 4) : dvp;
    L.kv = o, o += KT * kvw;
    L.p = o, o += apply ? rows * PS : 0;
    L.w = o, o += (apply && talk) ? rows * PS : 0;
    L.talk = o, o += (apply && talk) ? heads * heads : 0;
    L.m = o, o += apply ? rows : 0;
    L.l = o, o += apply ? rows : 0;
    o = (o + 1) & ~1;
    L.off = o, o += 2 * KT;   // KT 64-bit row offsets
    L.total = o;
    return L;
}

// cache rows [kb, kb + nk) of one key/value head -> dst[key][np] fp32 (zeros beyond n and beyond nk).  A thread issues
// the loads of eight pieces before it converts and stores any of them, so that they are in flight together.
template <typename T>
__device__ __forceinline__ void load_tile(const T* pool, const long long* rowoff, int nk, int head_off, int n, int np,
                                          int stride, float* dst, int vec) {
    constexpr int U = 8;
    const int n4 = np >> 2, total = KT * n4;
    for (int base = threadIdx.x; base < total; base += NT * U) {
        float4 v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int idx = base + u * NT;
            v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (idx >= total) continue;
            const int key = idx / n4, d = (idx - key * n4) << 2;
            if (key >= nk) continue;
            const T* src = pool + rowoff[key] + head_off + d;
            if (vec) {
                if constexpr (sizeof(T) == 2) {
                    const uint2 raw = *reinterpret_cast<const uint2*>(src);
                    v[u] = make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u),
                                       __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xffff0000u));
                } else {
                    v[u] = *reinterpret_cast<const float4*>(src);
                }
            } else {
                if (d + 0 < n) v[u].x = ldf(src + 0);
                if (d + 1 < n) v[u].y = ldf(src + 1);
                if (d + 2 < n) v[u].z = ldf(src + 2);
                if (d + 3 < n) v[u].w = ldf(src + 3);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int idx = base + u * NT;
            if (idx >= total) continue;
            const int key = idx / n4, d = (idx - key * n4) << 2;
            *reinterpret_cast<float4*>(dst + (size_t)key * stride + d) = v[u];
        }
    }
}

template <typename T, bool APPLY, int CB>
__global__ void __launch_bounds__(NT) mix_attn_kernel(MixArgs a) {
    extern __shared__ __align__(16) float sm[];
    const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    const int H = a.d.heads, G = a.d.kv_heads, rep = H / G, dk = a.d.dk, dv = a.d.dv, QT = a.QT, chunk = a.d.chunk;
    const int b = blockIdx.y;
    const int seq_end = a.cu_q[b + 1];
    const int q_beg = a.cu_q[b] + blockIdx.x * QT;
    if (q_beg >= seq_end) return;
    const int nq = min(QT, seq_end - q_beg);
    const int share = blockIdx.z % a.shares, gsel = blockIdx.z / a.shares;
    int gc0, gc1, hbeg, hend;
    if (!APPLY) {
        gc0 = gsel, gc1 = gsel + 1, hbeg = gc0 * rep, hend = gc1 * rep;
    } else {
        gc0 = gsel * a.gp, gc1 = min(G, gc0 + a.gp);
        if (a.talk)
            hbeg = 0, hend = H;
        else
            hbeg = gc0 * rep, hend = gc1 * rep;
    }
    const int rows = (hend - hbeg) * QT, Rg = rep * QT;
    const int dkp = a.dkp, dvp = a.dvp, KS = dkp + 4;
    const Layout L = mix_layout(rows, dkp, dvp, H, APPLY, a.talk != nullptr);
    float* qs = sm + L.q;
    float* kv = sm + L.kv;
    float* Pm = sm + L.p;
    float* Wm = a.talk ? sm + L.w : Pm;
    float* talk_s = sm + L.talk;
    float* Mr = sm + L.m;
    float* Lr = sm + L.l;
    long long* rowoff = reinterpret_cast<long long*>(sm + L.off);
    const int M = a.ix.M;
    const int p0 = a.ix.positions[q_beg], p1 = p0 + nq - 1;
    const int kmin = chunk > 0 ? (p0 / chunk) * chunk : 0;
    const int ntile = (p1 - kmin) / KT + 1;
    const int per = (ntile + a.shares - 1) / a.shares;
    const int t0 = share * per, t1 = min(ntile, t0 + per);
    const int slot = a.seq_slot[b];
    const T* pool = static_cast<const T*>(a.cache.pool);
    const int row_elems = G * (dk + dv), psz = a.cache.page_size;

    // queries of the CTA's heads: row (h - hbeg) * QT + i, zero padded
    for (int idx = tid; idx < rows * dkp; idx += NT) {
        const int row = idx / dkp, d = idx - row * dkp;
        const int h = hbeg + row / QT, i = row % QT;
        qs[idx] = (i < nq && d < dk) ? a.q[(long long)(q_beg + i) * a.ldq + (long long)h * dk + d] : 0.f;
    }
    if (APPLY) {
        if (a.talk)
            for (int i = tid; i < H * H; i += NT) talk_s[i] = a.talk[i];
        for (int row = tid; row < rows; row += NT) {   // final statistics: the key shares' maxima and sums merged
            const int h = hbeg + row / QT, i = row % QT;
            float mm = -INFINITY, ll = 0.f;
            if (i < nq) {
                const long long at = (long long)(q_beg + i) * H + h;
                for (int s = 0; s < a.shares; ++s) mm = fmaxf(mm, a.stats[(long long)s * M * H + at]);
                for (int s = 0; s < a.shares; ++s) {
                    const float ms = a.stats[(long long)s * M * H + at];
                    if (ms > -INFINITY) ll += a.stats[(long long)(a.shares + s) * M * H + at] * expf(ms - mm);
                }
            }
            Mr[row] = mm > -INFINITY ? mm : 0.f;
            Lr[row] = ll > 0.f ? 1.f / ll : 0.f;
        }
    }
    float mrun[4][2], lrun[4][2];
    float o[SLOTS][CB][4];
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int x = 0; x < 2; ++x) mrun[r][x] = -INFINITY, lrun[r][x] = 0.f;
#pragma unroll
    for (int s = 0; s < SLOTS; ++s)
#pragma unroll
        for (int c = 0; c < CB; ++c)
#pragma unroll
            for (int e = 0; e < 4; ++e) o[s][c][e] = 0.f;

    const int sc0 = (APPLY && a.talk) ? 0 : gc0, sc1 = (APPLY && a.talk) ? G : gc1;   // groups whose scores are needed
    for (int t = t0; t < t1; ++t) {
        const int kb = kmin + t * KT;
        const int nk = min(KT, p1 - kb + 1);
        __syncthreads();
        if (tid < KT) {
            long long off = 0;
            if (tid < nk) {
                const int j = kb + tid;
                const int page = a.cache.page_table[(long long)slot * a.cache.max_pages + j / psz];
                off = ((long long)page * psz + j % psz) * row_elems;
            }
            rowoff[tid] = off;
        }
        for (int c = sc0; c < sc1; ++c) {
            __syncthreads();
            load_tile<T>(pool, rowoff, nk, c * dk, dk, dkp, KS, kv, a.vec);
            __syncthreads();
            const int lrow0 = (c * rep - hbeg) * QT;   // first CTA row of this group
#pragma unroll
            for (int rc = 0; rc < 4; ++rc) {
                if (rc * 32 >= Rg) break;
                const int rg0 = rc * 32 + ty, rg1 = rg0 + 16;
                const float* qa = qs + (size_t)(lrow0 + min(rg0, Rg - 1)) * dkp;
                const float* qb = qs + (size_t)(lrow0 + min(rg1, Rg - 1)) * dkp;
                float acc[2][4];
#pragma unroll
                for (int x = 0; x < 2; ++x)
#pragma unroll
                    for (int y = 0; y < 4; ++y) acc[x][y] = 0.f;
                for (int d = 0; d < dkp; d += 4) {
                    const float4 a0 = *reinterpret_cast<const float4*>(qa + d);
                    const float4 a1 = *reinterpret_cast<const float4*>(qb + d);
#pragma unroll
                    for (int y = 0; y < 4; ++y) {
                        const float4 kk = *reinterpret_cast<const float4*>(kv + (size_t)(tx + 16 * y) * KS + d);
                        acc[0][y] = fmaf(a0.x, kk.x, acc[0][y]);
                        acc[0][y] = fmaf(a0.y, kk.y, acc[0][y]);
                        acc[0][y] = fmaf(a0.z, kk.z, acc[0][y]);
                        acc[0][y] = fmaf(a0.w, kk.w, acc[0][y]);
                        acc[1][y] = fmaf(a1.x, kk.x, acc[1][y]);
                        acc[1][y] = fmaf(a1.y, kk.y, acc[1][y]);
                        acc[1][y] = fmaf(a1.z, kk.z, acc[1][y]);
                        acc[1][y] = fmaf(a1.w, kk.w, acc[1][y]);
                    }
                }
#pragma unroll
                for (int x = 0; x < 2; ++x) {
                    const int rg = x ? rg1 : rg0;
                    const bool row_ok = rg < Rg;
                    const int hh = row_ok ? rg / QT : 0, i = row_ok ? rg % QT : 0;
                    const int h = c * rep + hh, pos = p0 + i;
                    const int lo = chunk > 0 ? (pos / chunk) * chunk : 0;
                    float s[4];
                    float tmax = -INFINITY;
#pragma unroll
                    for (int y = 0; y < 4; ++y) {
                        const int jj = tx + 16 * y, j = kb + jj;
                        const bool ok = row_ok && i < nq && jj < nk && j <= pos && j >= lo;
                        float v = acc[x][y] * a.d.scale;
                        if (a.dist_bias && ok) v += a.dist_bias[(long long)min(pos - j, a.far) * H + h];
                        s[y] = ok ? v : -INFINITY;
                        tmax = fmaxf(tmax, s[y]);
                    }
                    if (!APPLY) {
#pragma unroll
                        for (int w = 8; w > 0; w >>= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, w));
                        const float mnew = fmaxf(mrun[rc][x], tmax);
                        float sum = 0.f;
                        if (mnew > -INFINITY) {
#pragma unroll
                            for (int y = 0; y < 4; ++y) sum += s[y] > -INFINITY ? expf(s[y] - mnew) : 0.f;
                        }
#pragma unroll
                        for (int w = 8; w > 0; w >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, w);
                        if (mnew > -INFINITY) {
                            const float keep = mrun[rc][x] > -INFINITY ? expf(mrun[rc][x] - mnew) : 0.f;
                            lrun[rc][x] = lrun[rc][x] * keep + sum;
                            mrun[rc][x] = mnew;
                        }
                    } else if (row_ok) {
                        const int lrow = lrow0 + rg;
                        const float mm = Mr[lrow], il = Lr[lrow];
#pragma unroll
                        for (int y = 0; y < 4; ++y)
                            Pm[(size_t)lrow * PS + tx + 16 * y] = s[y] > -INFINITY ? expf(s[y] - mm) * il : 0.f;
                    }
                }
            }
        }
        if (!APPLY) continue;
        __syncthreads();
        if (a.talk) {   // w'_h = sum_g talk[h][g] w_g for the heads whose values this CTA multiplies
            const int h0 = gc0 * rep, h1 = gc1 * rep;
            for (int idx = tid; idx < QT * KT; idx += NT) {
                const int i = idx / KT, j = idx - i * KT;
                for (int h = h0; h < h1; ++h) {
                    float acc = 0.f;
                    for (int g = 0; g < H; ++g) acc = fmaf(talk_s[h * H + g], Pm[(size_t)(g * QT + i) * PS + j], acc);
                    Wm[(size_t)(h * QT + i) * PS + j] = acc;
                }
            }
        }
        for (int c = gc0; c < gc1; ++c) {
            __syncthreads();
            load_tile<T>(pool, rowoff, nk, G * dk + c * dv, dv, dvp, dvp, kv, a.vec);
            __syncthreads();
            const int cl = c - gc0;
            const int lrow0 = (c * rep - hbeg) * QT;
            const float* wrow[SLOTS];
            bool active[SLOTS];
#pragma unroll
            for (int s = 0; s < SLOTS; ++s) {
                const int rg = ty + 16 * (s % a.rag);
                active[s] = (s / a.rag == cl) && rg < Rg;
                wrow[s] = Wm + (size_t)(lrow0 + (active[s] ? rg : 0)) * PS;
            }
            for (int j = 0; j < nk; ++j) {
                float4 v[CB];
#pragma unroll
                for (int cb = 0; cb < CB; ++cb)
                    v[cb] = (cb * 64 + tx * 4) < dvp ? *reinterpret_cast<const float4*>(kv + (size_t)j * dvp + cb * 64 + tx * 4)
                                                     : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int s = 0; s < SLOTS; ++s) {
                    if (!active[s]) continue;
                    const float w = wrow[s][j];
#pragma unroll
                    for (int cb = 0; cb < CB; ++cb) {
                        o[s][cb][0] = fmaf(w, v[cb].x, o[s][cb][0]);
                        o[s][cb][1] = fmaf(w, v[cb].y, o[s][cb][1]);
                        o[s][cb][2] = fmaf(w, v[cb].z, o[s][cb][2]);
                        o[s][cb][3] = fmaf(w, v[cb].w, o[s][cb][3]);
                    }
                }
            }
        }
    }

    if (!APPLY) {
        if (tx == 0) {
#pragma unroll
            for (int rc = 0; rc < 4; ++rc)
#pragma unroll
                for (int x = 0; x < 2; ++x) {
                    const int rg = rc * 32 + ty + 16 * x;
                    if (rg >= Rg) continue;
                    const int hh = rg / QT, i = rg % QT;
                    if (i >= nq) continue;
                    const long long at = (long long)(q_beg + i) * H + gc0 * rep + hh;
                    a.stats[(long long)share * M * H + at] = mrun[rc][x];
                    a.stats[(long long)(a.shares + share) * M * H + at] = lrun[rc][x];
                }
        }
        return;
    }
#pragma unroll
    for (int s = 0; s < SLOTS; ++s) {
        const int cl = s / a.rag, c = gc0 + cl, rg = ty + 16 * (s % a.rag);
        if (c >= gc1 || rg >= Rg) continue;
        const int hh = rg / QT, i = rg % QT, h = c * rep + hh;
        if (i >= nq) continue;
        const int m = q_beg + i;
        float gate = 1.f;
        if (a.shares == 1 && a.gate) gate = 1.f / (1.f + expf(-a.gate[(long long)m * a.ldg + h]));
#pragma unroll
        for (int cb = 0; cb < CB; ++cb)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int col = cb * 64 + tx * 4 + e;
                if (col >= dv) continue;
                if (a.shares == 1)
                    stx(a.out, (long long)m * a.ldo + (long long)h * dv + col, a.of32, o[s][cb][e] * gate);
                else
                    a.part[((long long)share * M + m) * H * dv + (long long)h * dv + col] = o[s][cb][e];
            }
    }
}

// out[m][h][:] = sigmoid(gate[m][h]) * sum over the key shares (in index order) of their partial results
__global__ void mix_merge_kernel(const float* part, int shares, int M, int H, int dv, const float* gate, long long ldg,
                                 void* out, int of32, long long ldo) {
    const int m = blockIdx.x, n = H * dv;
    const int e = blockIdx.y * blockDim.x + threadIdx.x;
    if (e >= n) return;
    float acc = 0.f;
#pragma unroll 8
    for (int s = 0; s < shares; ++s) acc += part[((long long)s * M + m) * n + e];
    const int h = e / dv;
    if (gate) acc *= 1.f / (1.f + expf(-gate[(long long)m * ldg + h]));
    stx(out, (long long)m * ldo + e, of32, acc);
}

// ---------------------------------------------------------------------------------------------- steps of few tokens
// Every token on its own (its position and slot), its keys cut into shares: grid (shares, tokens).  The scores are
// computed once, by all threads over 64 keys x 4 heads at a time, and kept in the workspace (a few hundred KB per token
// beside megabytes of cache rows); the second kernel reads them back, so keys are read once and values once.
constexpr int DEC_OA = 8;   // heads of one key/value group a thread accumulates in the second kernel

struct DecLayout {
    int q, kv, p, w, os, talk, m, l, off, total;   // float offsets
};
// sk: keys a share holds at most (second kernel)
__host__ __device__ inline DecLayout dec_layout(int H, int dkp, int dvp, bool apply, bool talk, int sk) {
    DecLayout L;
    int o = 0;
    L.q = o, o += apply ? 0 : H * dkp;
    L.kv = o;                                            // (no tile is staged)
    L.p = o, o += (apply && talk) ? H * KT : 0;
    L.w = o, o += apply ? H * sk : 0;
    L.os = o, o += apply ? (NT / 32) * DEC_OA * dvp : 0;     // the warps' sums of one key/value group
    L.talk = o, o += (apply && talk) ? H * H : 0;
    L.m = o, o += apply ? H : 0;
    L.l = o, o += apply ? H : 0;
    o = (o + 3) & ~3;
    L.off = o, o += 2 * (sk > KT ? sk : KT);   // 64-bit row offsets of the share's keys
    L.total = o;
    return L;
}

// eight consecutive elements of a cache row as floats (vec: one 16-byte load, or two for fp32 rows; else element by
// element with zeros from n on)
template <typename T>
__device__ __forceinline__ void load8(const T* src, int d, int n, int vec, float (&v)[8]) {
    if (vec && d + 8 <= n) {
        if constexpr (sizeof(T) == 2) {
            const uint4 raw = *reinterpret_cast<const uint4*>(src);
            v[0] = __uint_as_float(raw.x << 16), v[1] = __uint_as_float(raw.x & 0xffff0000u);
            v[2] = __uint_as_float(raw.y << 16), v[3] = __uint_as_float(raw.y & 0xffff0000u);
            v[4] = __uint_as_float(raw.z << 16), v[5] = __uint_as_float(raw.z & 0xffff0000u);
            v[6] = __uint_as_float(raw.w << 16), v[7] = __uint_as_float(raw.w & 0xffff0000u);
        } else {
            const float4 a = *reinterpret_cast<const float4*>(src), b = *reinterpret_cast<const float4*>(src + 4);
            v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
        }
    } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = d + e < n ? ldf(src + e) : 0.f;
    }
}

// cache row offsets of the share's keys [k0, k1) (relative to kmin) into rowoff[0 .. k1 - k0)
__device__ __forceinline__ void share_rows(const MixArgs& a, int slot, int kmin, int k0, int k1, int row_elems, long long* rowoff) {
    const int psz = a.cache.page_size;
    for (int i = threadIdx.x; i < k1 - k0; i += NT) {
        const int j = kmin + k0 + i;
        const int page = a.cache.page_table[(long long)slot * a.cache.max_pages + j / psz];
        rowoff[i] = ((long long)page * psz + j % psz) * row_elems;
    }
}

// First kernel.  Nothing is staged: eight lanes share a key row (16-byte pieces, whole lines per warp), a warp four
// keys at a time, against the queries of the key's group in shared memory; the partial dot products of the group's heads
// are closed by shuffles.
template <typename T>
__global__ void __launch_bounds__(NT) mix_dec_scores_kernel(MixArgs a) {
    extern __shared__ __align__(16) float sm[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, l8 = lane & 7, sub = lane >> 3;
    const int H = a.d.heads, G = a.d.kv_heads, rep = H / G, dk = a.d.dk, dv = a.d.dv, chunk = a.d.chunk;
    const int m = blockIdx.y, share = blockIdx.x, M = a.ix.M;
    const int dkp = a.dkp, SK = a.rag;
    const DecLayout L = dec_layout(H, dkp, a.dvp, false, false, SK);
    float* qs = sm + L.q;
    long long* rowoff = reinterpret_cast<long long*>(sm + L.off);
    const int pos = a.ix.positions[m], slot = a.ix.token_slot[m];
    const int kmin = chunk > 0 ? (pos / chunk) * chunk : 0;
    const int n = pos - kmin + 1, ntile = (n + KT - 1) / KT;
    const int per = (ntile + a.shares - 1) / a.shares;
    const int k0 = min(n, share * per * KT), k1 = min(n, (share + 1) * per * KT);
    const T* pool = static_cast<const T*>(a.cache.pool);
    const int row_elems = G * (dk + dv);
    float* srow = a.scores + (long long)m * H * a.score_ld;
    for (int idx = tid; idx < H * dkp; idx += NT) {
        const int h = idx / dkp, d = idx - h * dkp;
        qs[idx] = d < dk ? a.q[(long long)m * a.ldq + (long long)h * dk + d] : 0.f;
    }
    share_rows(a, slot, kmin, k0, k1, row_elems, rowoff);
    __syncthreads();
    const int npiece = dkp >> 3, nkey = k1 - k0;
    for (int c = 0; c < G; ++c) {
        const float* qg = qs + (size_t)c * rep * dkp;
#pragma unroll 2
        for (int kq = warp * 4; kq < nkey; kq += (NT / 32) * 4) {
            const int ki = kq + sub;
            const bool live = ki < nkey;
            const T* kr = pool + rowoff[live ? ki : 0] + c * dk;
            float acc[DEC_OA];
#pragma unroll
            for (int x = 0; x < DEC_OA; ++x) acc[x] = 0.f;
            for (int p = l8; p < npiece; p += 8) {
                float kk[8];
                load8<T>(kr + 8 * p, 8 * p, dk, a.gp, kk);
#pragma unroll
                for (int x = 0; x < DEC_OA; ++x) {
                    if (x >= rep) break;
                    const float4 q0 = *reinterpret_cast<const float4*>(qg + (size_t)x * dkp + 8 * p);
                    const float4 q1 = *reinterpret_cast<const float4*>(qg + (size_t)x * dkp + 8 * p + 4);
                    acc[x] = fmaf(q0.x, kk[0], acc[x]);
                    acc[x] = fmaf(q0.y, kk[1], acc[x]);
                    acc[x] = fmaf(q0.z, kk[2], acc[x]);
                    acc[x] = fmaf(q0.w, kk[3], acc[x]);
                    acc[x] = fmaf(q1.x, kk[4], acc[x]);
                    acc[x] = fmaf(q1.y, kk[5], acc[x]);
                    acc[x] = fmaf(q1.z, kk[6], acc[x]);
                    acc[x] = fmaf(q1.w, kk[7], acc[x]);
                }
            }
#pragma unroll
            for (int x = 0; x < DEC_OA; ++x) {
                if (x >= rep) break;
                float v = acc[x];
                v += __shfl_xor_sync(0xffffffffu, v, 1);
                v += __shfl_xor_sync(0xffffffffu, v, 2);
                v += __shfl_xor_sync(0xffffffffu, v, 4);
                if (l8 == 0 && live) {
                    const int h = c * rep + x;
                    v *= a.d.scale;
                    if (a.dist_bias) v += a.dist_bias[(long long)min(pos - (kmin + k0 + ki), a.far) * H + h];
                    srow[(long long)h * a.score_ld + k0 + ki] = v;
                }
            }
        }
    }
    __syncthreads();
    // maximum and sum of exponentials of this share, head by head
    for (int h = warp; h < H; h += NT / 32) {
        const float* r = srow + (long long)h * a.score_ld;
        float mx = -INFINITY;
        for (int j = k0 + lane; j < k1; j += 32) mx = fmaxf(mx, r[j]);
        mx = warp_max(mx);
        float sum = 0.f;
        for (int j = k0 + lane; j < k1; j += 32) sum += expf(r[j] - mx);
        sum = warp_sum(sum);
        if (lane == 0) {
            const long long at = (long long)m * H + h;
            a.stats[(long long)share * M * H + at] = mx;
            a.stats[(long long)(a.shares + share) * M * H + at] = k1 > k0 ? sum : 0.f;
        }
    }
}

// Second kernel: the share's normalised, mixed weights for ALL its keys first (shared memory, [heads][keys of the share]),
// then one key/value group after the other: a warp takes every eighth key of a value tile, a lane four value columns,
// so a value is read once for all heads of its group; the warps' sums are added in index order.
template <typename T>
__global__ void __launch_bounds__(NT) mix_dec_apply_kernel(MixArgs a) {
    extern __shared__ __align__(16) float sm[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int H = a.d.heads, G = a.d.kv_heads, rep = H / G, dk = a.d.dk, dv = a.d.dv, chunk = a.d.chunk;
    const int m = blockIdx.y, share = blockIdx.x, M = a.ix.M;
    const int dvp = a.dvp, SK = a.rag;       // keys a share holds at most (a multiple of the tile)
    const bool talk = a.talk != nullptr;
    const DecLayout L = dec_layout(H, a.dkp, dvp, true, talk, SK);
    float* kv = sm + L.kv;
    float* Pm = sm + L.p;
    float* Wm = sm + L.w;
    float* red = sm + L.os;
    float* talk_s = sm + L.talk;
    float* Mh = sm + L.m;
    float* Lh = sm + L.l;
    long long* rowoff = reinterpret_cast<long long*>(sm + L.off);
    const int pos = a.ix.positions[m], slot = a.ix.token_slot[m];
    const int kmin = chunk > 0 ? (pos / chunk) * chunk : 0;
    const int n = pos - kmin + 1, ntile = (n + KT - 1) / KT;
    const int per = (ntile + a.shares - 1) / a.shares;
    const int t0 = share * per, t1 = min(ntile, t0 + per);
    const T* pool = static_cast<const T*>(a.cache.pool);
    const int row_elems = G * (dk + dv), psz = a.cache.page_size;
    const float* srow = a.scores + (long long)m * H * a.score_ld;
    if (talk)
        for (int i = tid; i < H * H; i += NT) talk_s[i] = a.talk[i];
    for (int h = tid; h < H; h += NT) {
        const long long at = (long long)m * H + h;
        float mm = -INFINITY, ll = 0.f;
        for (int s = 0; s < a.shares; ++s) mm = fmaxf(mm, a.stats[(long long)s * M * H + at]);
        for (int s = 0; s < a.shares; ++s) {
            const float ms = a.stats[(long long)s * M * H + at];
            if (ms > -INFINITY) ll += a.stats[(long long)(a.shares + s) * M * H + at] * expf(ms - mm);
        }
        Mh[h] = mm > -INFINITY ? mm : 0.f;
        Lh[h] = ll > 0.f ? 1.f / ll : 0.f;
    }
    // weights of the share's keys
    for (int t = t0; t < t1; ++t) {
        const int kb = kmin + t * KT;
        const int nk = min(KT, pos - kb + 1);
        __syncthreads();
        float* dstp = talk ? Pm : Wm + (t - t0) * KT;
        const int ldp = talk ? KT : SK;
#pragma unroll 4
        for (int idx = tid; idx < H * KT; idx += NT) {
            const int h = idx / KT, jj = idx - h * KT;
            dstp[h * ldp + jj] = jj < nk ? expf(srow[(long long)h * a.score_ld + (kb - kmin) + jj] - Mh[h]) * Lh[h] : 0.f;
        }
        if (talk) {
            __syncthreads();
            for (int idx = tid; idx < H * KT; idx += NT) {
                const int h = idx / KT, jj = idx - h * KT;
                float acc = 0.f;
                for (int g = 0; g < H; ++g) acc = fmaf(talk_s[h * H + g], Pm[g * KT + jj], acc);
                Wm[h * SK + (t - t0) * KT + jj] = acc;
            }
        }
    }
    const bool col_ok = 4 * lane < dvp;
    const int k0 = min(n, t0 * KT), k1 = min(n, t1 * KT), nkey = k1 - k0;
    __syncthreads();
    share_rows(a, slot, kmin, k0, k1, row_elems, rowoff);
    __syncthreads();
    for (int c = 0; c < G; ++c) {
        float acc[DEC_OA][4];
#pragma unroll
        for (int x = 0; x < DEC_OA; ++x)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[x][e] = 0.f;
        if (col_ok) {   // nothing staged: a warp reads a key's value row (four columns a lane), every eighth key
            const float* wbase = Wm + (size_t)(c * rep) * SK;
            const int voff = G * dk + c * dv + 4 * lane;
            for (int kb = warp; kb < nkey; kb += (NT / 32) * 4) {
                float4 v[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int ki = kb + u * (NT / 32);
                    v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (ki >= nkey) continue;
                    const T* src = pool + rowoff[ki] + voff;
                    if (a.vec) {
                        if constexpr (sizeof(T) == 2) {
                            const uint2 raw = *reinterpret_cast<const uint2*>(src);
                            v[u] = make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u),
                                               __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xffff0000u));
                        } else {
                            v[u] = *reinterpret_cast<const float4*>(src);
                        }
                    } else {
                        if (4 * lane + 0 < dv) v[u].x = ldf(src + 0);
                        if (4 * lane + 1 < dv) v[u].y = ldf(src + 1);
                        if (4 * lane + 2 < dv) v[u].z = ldf(src + 2);
                        if (4 * lane + 3 < dv) v[u].w = ldf(src + 3);
                    }
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int ki = kb + u * (NT / 32);
                    if (ki >= nkey) continue;
#pragma unroll
                    for (int x = 0; x < DEC_OA; ++x) {
                        if (x >= rep) break;
                        const float w = wbase[(size_t)x * SK + ki];
                        acc[x][0] = fmaf(w, v[u].x, acc[x][0]);
                        acc[x][1] = fmaf(w, v[u].y, acc[x][1]);
                        acc[x][2] = fmaf(w, v[u].z, acc[x][2]);
                        acc[x][3] = fmaf(w, v[u].w, acc[x][3]);
                    }
                }
            }
        }
        __syncthreads();
        if (col_ok) {
#pragma unroll
            for (int x = 0; x < DEC_OA; ++x) {
                if (x >= rep) break;
                *reinterpret_cast<float4*>(red + ((size_t)warp * rep + x) * dvp + 4 * lane) =
                    make_float4(acc[x][0], acc[x][1], acc[x][2], acc[x][3]);
            }
        }
        __syncthreads();
        for (int idx = tid; idx < rep * dv; idx += NT) {
            const int x = idx / dv, col = idx - x * dv, h = c * rep + x;
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < NT / 32; ++w) v += red[((size_t)w * rep + x) * dvp + col];
            if (a.shares == 1) {
                const float gate = a.gate ? 1.f / (1.f + expf(-a.gate[(long long)m * a.ldg + h])) : 1.f;
                stx(a.out, (long long)m * a.ldo + (long long)h * dv + col, a.of32, v * gate);
            } else {
                a.part[((long long)share * M + m) * H * dv + (long long)h * dv + col] = v;
            }
        }
    }
}

// dynamic shared memory: the row (n floats) + per-head sums of squares and factors
template <typename T>
__global__ void mix_post_kernel(SeqIndex ix, float* qkv, long long ld, MixDims d, MixPost p, PagedRows cache) {
    extern __shared__ float sm[];
    const int H = d.heads, G = d.kv_heads, dk = d.dk, dv = d.dv;
    const int nq = H * dk, nk = G * dk, nv = G * dv, n = nq + nk + nv, units = H + 2 * G;
    float* row = sm;
    float* fac = sm + n;
    const int m = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nw = blockDim.x >> 5;
    float* src = qkv + (long long)m * ld;
    for (int i = tid; i < n; i += blockDim.x) row[i] = src[i] + (p.bias ? p.bias[i] : 0.f);
    __syncthreads();
    // sum of squares of every query head, key head and value head
    for (int u = warp; u < units; u += nw) {
        const int beg = u < H ? u * dk : (u < H + G ? nq + (u - H) * dk : nq + nk + (u - H - G) * dv);
        const int len = u < H + G ? dk : dv;
        float ss = 0.f;
        for (int i = lane; i < len; i += 32) ss += row[beg + i] * row[beg + i];
        ss = warp_sum(ss);
        if (lane == 0) fac[u] = ss;
    }
    __syncthreads();
    if (tid == 0) {
        const int pos = ix.positions[m];
        const float temp = p.temp_every > 0 ? 1.f + p.temp_coef * logf((float)((pos + 1) / p.temp_every) + 1.f) : 1.f;
        float wq = 0.f, wk = 0.f;
        if (p.norm_whole) {
            for (int u = 0; u < H; ++u) wq += fac[u];
            for (int u = 0; u < G; ++u) wk += fac[H + u];
            wq = 1.f / sqrtf(wq / (float)nq + p.eps), wk = 1.f / sqrtf(wk / (float)nk + p.eps);
        }
        for (int u = 0; u < H; ++u) {
            float f = !p.q_norm ? 1.f : (p.norm_whole ? wq : 1.f / sqrtf(fac[u] / (float)dk + p.eps));
            f *= temp;
            if (p.head_factor) f *= p.head_factor[u];
            fac[u] = f;
        }
        for (int u = 0; u < G; ++u)
            fac[H + u] = !p.k_norm ? 1.f : (p.norm_whole ? wk : 1.f / sqrtf(fac[H + u] / (float)dk + p.eps));
        for (int u = 0; u < G; ++u) fac[H + G + u] = p.v_unit ? 1.f / sqrtf(fac[H + G + u] / (float)dv + p.eps) : 1.f;
    }
    __syncthreads();
    const int pos = ix.positions[m], slot = ix.token_slot[m];
    const int page = cache.page_table[(long long)slot * cache.max_pages + pos / cache.page_size];
    T* dst = static_cast<T*>(cache.pool) + ((long long)page * cache.page_size + pos % cache.page_size) * (nk + nv);
    for (int i = tid; i < n; i += blockDim.x) {
        if (i < nq) {
            const float w = p.q_norm ? p.q_norm[p.norm_whole ? i : i % dk] : 1.f;
            src[i] = row[i] * fac[i / dk] * w;
        } else if (i < nq + nk) {
            const int e = i - nq;
            const float w = p.k_norm ? p.k_norm[p.norm_whole ? e : e % dk] : 1.f;
            stf(dst + e, row[i] * fac[H + e / dk] * w);
        } else {
            const int e = i - nq - nk;
            stf(dst + nk + e, row[i] * fac[H + G + e / dv]);
        }
    }
}

}  // namespace

int launch_mix_post(const SeqIndex& ix, float* qkv, long long ld, const MixDims& d, const MixPost& p,
                    const PagedRows& cache, cudaStream_t stream) {
    if (ix.M <= 0) return 0;
    const int n = d.heads * d.dk + d.kv_heads * (d.dk + d.dv), units = d.heads + 2 * d.kv_heads;
    const size_t smem = (size_t)(n + units) * sizeof(float);
    if (smem > 200 * 1024) return set_error("mix_post: a row of %d values does not fit shared memory", n);
    static PerDeviceOnce once;
    if (once.need()) {
        ASD_CUDA(cudaFuncSetAttribute(mix_post_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
        ASD_CUDA(cudaFuncSetAttribute(mix_post_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
    }
    if (cache.f32)
        mix_post_kernel<float><<<ix.M, 128, smem, stream>>>(ix, qkv, ld, d, p, cache);
    else
        mix_post_kernel<__nv_bfloat16><<<ix.M, 128, smem, stream>>>(ix, qkv, ld, d, p, cache);
    count_launch(1);
    ASD_CUDA(cudaGetLastError());
    return 0;
}

int launch_mix_merge(const MixArgs& a, cudaStream_t stream) {
    const dim3 grid(a.ix.M, (a.d.heads * a.d.dv + 255) / 256);
    mix_merge_kernel<<<grid, 256, 0, stream>>>(a.part, a.shares, a.ix.M, a.d.heads, a.d.dv, a.gate, a.ldg, a.out, a.of32, a.ldo);
    count_launch(1);
    ASD_CUDA(cudaGetLastError());
    return 0;
}

template <typename T>
static int launch_dec(const MixArgs& a, dim3 grid, size_t smem_scores, size_t smem_apply, cudaStream_t stream) {
    static PerDeviceOnce once;
    if (once.need()) {
        ASD_CUDA(cudaFuncSetAttribute(mix_dec_scores_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
        ASD_CUDA(cudaFuncSetAttribute(mix_dec_apply_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
    }
    mix_dec_scores_kernel<T><<<grid, NT, smem_scores, stream>>>(a);
    mix_dec_apply_kernel<T><<<grid, NT, smem_apply, stream>>>(a);
    count_launch(2);
    ASD_CUDA(cudaGetLastError());
    return 0;
}

int launch_mix_attention_decode(MixArgs a, int nseq, int max_kv_len, const MixWork& ws, cudaStream_t stream) {
    (void)nseq;
    const int H = a.d.heads, G = a.d.kv_heads, rep = H / G, M = a.ix.M;
    const int dkp = (a.d.dk + 7) & ~7, dvp = (a.d.dv + 3) & ~3;
    if (dvp > 128 || rep > DEC_OA || !ws.scores || !ws.stats) return 1;
    const long long score_ld = (max_kv_len + 3) & ~3;
    if ((long long)M * H * score_ld > ws.score_elems) return 1;
    const int key_tiles = (max_kv_len + KT - 1) / KT;
    int shares = (int)std::min<long long>((444 + M - 1) / M, (long long)std::max(1, key_tiles / 2));
    shares = std::max(1, std::min(shares, 32));
    // the second kernel keeps the weights of a share's keys in shared memory: more shares where they would not fit
    auto smem_apply = [&](int sh) {
        const int per = (key_tiles + sh - 1) / sh;
        return (size_t)dec_layout(H, dkp, dvp, true, a.talk != nullptr, per * KT).total * sizeof(float);
    };
    while (smem_apply(shares) > 160 * 1024 && shares < 64 && shares < key_tiles) ++shares;
    const size_t sm_s = (size_t)dec_layout(H, dkp, dvp, false, false, ((key_tiles + shares - 1) / shares) * KT).total * sizeof(float);
    const size_t sm_a = smem_apply(shares);
    if (sm_s > 200 * 1024 || sm_a > 200 * 1024) return 1;
    if (shares > 1 && (!ws.part || (long long)shares * M * H * a.d.dv > ws.part_elems)) return 1;
    if ((long long)2 * shares * M * H > ws.stats_elems) return 1;
    a.shares = shares, a.dkp = dkp, a.dvp = dvp, a.rag = ((key_tiles + shares - 1) / shares) * KT, a.score_ld = score_ld;
    a.scores = ws.scores;
    a.vec = (a.d.dk % 4 == 0 && a.d.dv % 4 == 0) ? 1 : 0;                       // a lane's four value columns in one load
    const int piece = a.cache.f32 ? 4 : 8;                                       // elements of a 16-byte load
    a.gp = (a.d.dk % piece == 0 && a.d.dv % piece == 0) ? 1 : 0;                 // a lane's eight key elements in 16-byte loads
    const dim3 grid(shares, M);
    const int rc = a.cache.f32 ? launch_dec<float>(a, grid, sm_s, sm_a, stream)
                               : launch_dec<__nv_bfloat16>(a, grid, sm_s, sm_a, stream);
    if (rc) return -1;
    if (shares > 1 && launch_mix_merge(a, stream)) return -1;
    return 0;
}

template <typename T, bool APPLY, int CB>
static int launch_one(const MixArgs& a, dim3 grid, size_t smem, cudaStream_t stream) {
    static PerDeviceOnce once;
    if (once.need())
        ASD_CUDA(cudaFuncSetAttribute(mix_attn_kernel<T, APPLY, CB>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
    mix_attn_kernel<T, APPLY, CB><<<grid, NT, smem, stream>>>(a);
    count_launch(1);
    ASD_CUDA(cudaGetLastError());
    return 0;
}

int mix_attention_check(const MixDims& d, int talk) {
    if (d.heads <= 0 || d.kv_heads <= 0 || d.heads % d.kv_heads || d.dk <= 0 || d.dv <= 0 || d.chunk < 0)
        return set_error("mixed attention: bad sizes");
    if (d.dv > 256) return set_error("mixed attention: value size %d above 256", d.dv);
    if (d.dk > 512) return set_error("mixed attention: key size %d above 512", d.dk);
    if (d.heads / d.kv_heads > MAX_ROWS) return set_error("mixed attention: more than %d query heads per key head", MAX_ROWS);
    if (talk && d.heads > MAX_ROWS) return set_error("mixed attention: more than %d heads with mixed weights", MAX_ROWS);
    return 0;
}

int launch_mix_attention(const SeqIndex& ix, const int* cu_q, const int* seq_slot, int nseq, int max_qlen, int max_kv_len,
                         const float* q, long long ldq, const MixDims& d, const float* dist_bias, int far,
                         const float* talk, const float* gate, long long ldg, const PagedRows& cache, void* out, int of32,
                         long long ldo, const MixWork& ws, cudaStream_t stream) {
    if (ix.M <= 0 || nseq <= 0) return 0;
    if (mix_attention_check(d, talk != nullptr)) return -1;
    const int H = d.heads, G = d.kv_heads, rep = H / G;
    const int dkp = (d.dk + 3) & ~3, dvp = (d.dv + 3) & ~3;
    MixArgs a;
    a.ix = ix, a.cu_q = cu_q, a.seq_slot = seq_slot, a.q = q, a.ldq = ldq, a.d = d, a.dist_bias = dist_bias, a.far = far;
    a.talk = talk, a.gate = gate, a.ldg = ldg, a.cache = cache, a.out = out, a.of32 = of32, a.ldo = ldo;
    a.stats = ws.stats, a.part = ws.part, a.dkp = dkp, a.dvp = dvp, a.scores = nullptr, a.score_ld = 0;
    a.QT = 1, a.shares = 1, a.gp = 1, a.rag = 1;
    a.vec = (d.dk % 4 == 0 && d.dv % 4 == 0) ? 1 : 0;
    // steps of few tokens; prompts of a bf16 engine on the tensor cores; else (and for sizes those refuse) the CUDA cores
    if (max_qlen <= 4 && ws.mode != 1) {
        const int rc = launch_mix_attention_decode(a, nseq, max_kv_len, ws, stream);
        if (rc <= 0) return rc;
    }
    if (!cache.f32 && ws.mode != 1) {
        const int rc = launch_mix_attention_tc(a, nseq, max_qlen, max_kv_len, ws, stream);
        if (rc <= 0) return rc;
    }
    // key/value groups per apply CTA and queries per tile: the CTA's (head, query) pairs, the result rows a thread
    // holds and shared memory must fit
    const int want_qt = max_qlen >= 16 ? 16 : (max_qlen >= 8 ? 8 : (max_qlen >= 4 ? 4 : (max_qlen >= 2 ? 2 : 1)));
    int gp = talk ? G : 1, QT = 0;
    size_t smem_apply = 0;
    for (; gp >= 1 && !QT; gp = (gp + 1) / 2) {
        for (int qt = want_qt; qt >= 1; qt >>= 1) {
            const int rows = (talk ? H : gp * rep) * qt, rag = (rep * qt + 15) / 16;
            const size_t sm = (size_t)mix_layout(rows, dkp, dvp, H, true, talk != nullptr).total * sizeof(float);
            if (rows <= MAX_ROWS && rep * qt <= MAX_ROWS && gp * rag <= SLOTS && sm <= 200 * 1024) {
                QT = qt, smem_apply = sm;
                break;
            }
        }
        if (QT || gp == 1) break;
    }
    if (!QT) return set_error("mixed attention: %d heads of %d + %d values do not fit a CTA", H, d.dk, d.dv);
    a.QT = QT, a.gp = gp, a.rag = (rep * QT + 15) / 16;
    const int tiles = (max_qlen + QT - 1) / QT, ngroups = (G + gp - 1) / gp;
    // steps of few tokens: cut the keys into shares so that the CTAs cover the SMs
    int shares = 1;
    const long long base = (long long)tiles * nseq * ngroups;
    const int key_tiles = (max_kv_len + KT - 1) / KT;
    if (base < 148 && ws.stats && ws.part) {
        shares = (int)std::min<long long>((296 + base - 1) / base, (long long)std::max(1, key_tiles / 2));
        shares = std::min(shares, 32);
        while (shares > 1 && ((long long)shares * ix.M * H * d.dv > ws.part_elems ||
                              (long long)2 * shares * ix.M * H > ws.stats_elems))
            --shares;
    }
    if ((long long)2 * shares * ix.M * H > ws.stats_elems || !ws.stats)
        return set_error("mixed attention: statistics workspace too small");
    a.shares = shares;
    const size_t smem_stats = (size_t)mix_layout(rep * QT, dkp, dvp, H, false, false).total * sizeof(float);
    const dim3 gs(tiles, nseq, shares * G), ga(tiles, nseq, shares * ngroups);
    const int cb = dvp <= 64 ? 1 : (dvp <= 128 ? 2 : 4);
    int rc;
    if (cache.f32) {
        rc = launch_one<float, false, 1>(a, gs, smem_stats, stream);
        if (!rc)
            rc = cb == 1 ? launch_one<float, true, 1>(a, ga, smem_apply, stream)
                         : (cb == 2 ? launch_one<float, true, 2>(a, ga, smem_apply, stream)
                                    : launch_one<float, true, 4>(a, ga, smem_apply, stream));
    } else {
        rc = launch_one<__nv_bfloat16, false, 1>(a, gs, smem_stats, stream);
        if (!rc)
            rc = cb == 1 ? launch_one<__nv_bfloat16, true, 1>(a, ga, smem_apply, stream)
                         : (cb == 2 ? launch_one<__nv_bfloat16, true, 2>(a, ga, smem_apply, stream)
                                    : launch_one<__nv_bfloat16, true, 4>(a, ga, smem_apply, stream));
    }
    if (rc) return rc;
    if (shares > 1) {
        if (launch_mix_merge(a, stream)) return -1;
    }
    return 0;
}

}  // namespace asd
