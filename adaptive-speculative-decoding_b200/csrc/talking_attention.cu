// Talking-heads window attention: grouped-query softmax attention over a sliding window whose scores pass a tanh cap and
// are then mixed across the heads (s'_h = sum_g talk[h][g] s_g) before a softmax with a sink per head in its denominator.
// The mix needs every head's score of a (query, key) pair, so one CTA serves ALL heads of a tile of query positions.
// talk_post_kernel:  biases, RMS norm of every query / key head (plain weight), rotation of the leading coordinates in
//   pairs (2 i, 2 i + 1), queries left in place, keys and values appended to the paged cache; one warp per (token, head).
// talk_attention_kernel: one CTA per (sequence, TQ consecutive new positions), one warp per head.  Keys are visited in
//   tiles of TK positions that start at multiples of TK (a position's sums run over the same tiles in the same order
//   however its sequence was cut into forwards): the tile's cache rows are copied in 16-byte pieces, several in flight
//   per lane, and staged in shared memory as fp32 once for all heads and all TQ queries; lane = key for the scores (a
//   key coordinate is read once for the TQ queries; capped, stored for the other heads), then every warp mixes its
//   head's row, folds it into the running softmax (which starts from the sink: maximum = sink, sum = 1, nothing
//   accumulated) and adds the values with lane = value column (a value is read once for the TQ queries).
#include <cuda_bf16.h>
#include <math.h>

#include "asd_internal.h"
#include "blocks.h"
#include "elem.cuh"
#include "mma_sync.cuh"

namespace asd {

namespace {

__device__ __forceinline__ long long cache_row(const PagedRows& c, int slot, int pos) {
    const int page = c.page_table[(long long)slot * c.max_pages + pos / c.page_size];
    return (long long)page * c.page_size + pos % c.page_size;
}

__global__ void talk_post_kernel(SeqIndex ix, float* qkv, long long ld, TalkDims d, const float* bias, const float* q_norm,
                                 const float* k_norm, float eps, const float* freq, PagedRows cache) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int units = d.heads + 2 * d.kv_heads;
    const long long idx = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
    if (idx >= (long long)ix.M * units) return;
    const int m = (int)(idx / units), u = (int)(idx - (long long)m * units);
    const int pos = ix.positions[m];
    const int row_elems = d.kv_heads * (d.dk + d.dv);
    const long long crow = cache_row(cache, ix.token_slot[m], pos) * row_elems;
    if (u >= d.heads + d.kv_heads) {   // a value head: bias, then the cache
        const int g = u - d.heads - d.kv_heads;
        const int off = (d.heads + d.kv_heads) * d.dk + g * d.dv;
        const float* src = qkv + (long long)m * ld + off;
        for (int i = lane; i < d.dv; i += 32)
            stx(cache.pool, crow + (long long)d.kv_heads * d.dk + g * d.dv + i, cache.f32, src[i] + (bias ? bias[off + i] : 0.f));
        return;
    }
    const bool is_q = u < d.heads;
    const int off = u * d.dk;          // queries, then keys
    float* src = qkv + (long long)m * ld + off;
    const float* w = is_q ? q_norm : k_norm;
    float ss = 0.f;
    for (int i = lane; i < d.dk; i += 32) {
        const float v = src[i] + (bias ? bias[off + i] : 0.f);
        ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    const float r = w ? 1.f / sqrtf(ss / (float)d.dk + eps) : 1.f;
    for (int e = 2 * lane; e < d.dk; e += 64) {
        float a = (src[e] + (bias ? bias[off + e] : 0.f)) * r * (w ? w[e] : 1.f);
        const bool two = e + 1 < d.dk;
        float b = two ? (src[e + 1] + (bias ? bias[off + e + 1] : 0.f)) * r * (w ? w[e + 1] : 1.f) : 0.f;
        if (e + 1 < d.rot_dims) {
            float sn, cs;
            sincosf((float)pos * freq[e >> 1], &sn, &cs);
            const float ra = a * cs - b * sn, rb = b * cs + a * sn;
            a = ra, b = rb;
        }
        if (is_q) {
            src[e] = a;
            if (two) src[e + 1] = b;
        } else {
            const long long dst = crow + (long long)(u - d.heads) * d.dk + e;
            stx(cache.pool, dst, cache.f32, a);
            if (two) stx(cache.pool, dst + 1, cache.f32, b);
        }
    }
}

struct TalkTile {
    int tk;                // key positions per tile (<= 32)
    int ks_stride;         // floats per staged key row (odd: lanes = keys read without bank conflicts)
    int vec;               // 1: cache rows are copied in 16-byte pieces
};

// one cache row (keys, then values) -> fp32 in shared memory, 16 bytes per lane and load, four loads in flight
template <typename T>
__device__ __forceinline__ void stage_row_vec(const T* row, bool valid, float* kdst, float* vdst, int nk, int nv, int lane) {
    constexpr int VE = 16 / sizeof(T);
    const int nvec = (nk + nv) / VE;
    for (int v0 = lane; v0 < nvec; v0 += 128) {
        uint4 r[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int v = v0 + 32 * u;
            r[u] = (valid && v < nvec) ? __ldg(reinterpret_cast<const uint4*>(row) + v) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int v = v0 + 32 * u;
            if (v >= nvec) continue;
            const int e = v * VE;
            float* dst = e < nk ? kdst + e : vdst + (e - nk);
            const T* x = reinterpret_cast<const T*>(&r[u]);
#pragma unroll
            for (int i = 0; i < VE; ++i) dst[i] = (float)x[i];
        }
    }
}

// TQ consecutive floats from shared memory (16-byte aligned for TQ >= 4, 8-byte for TQ = 2) in as few loads as possible
template <int TQ>
__device__ __forceinline__ void load_tq(const float* p, float (&r)[TQ]) {
    if constexpr (TQ % 4 == 0) {
#pragma unroll
        for (int i = 0; i < TQ / 4; ++i) {
            const float4 v = reinterpret_cast<const float4*>(p)[i];
            r[4 * i] = v.x, r[4 * i + 1] = v.y, r[4 * i + 2] = v.z, r[4 * i + 3] = v.w;
        }
    } else if constexpr (TQ == 2) {
        const float2 v = *reinterpret_cast<const float2*>(p);
        r[0] = v.x, r[1] = v.y;
    } else {
        r[0] = p[0];
    }
}

// TQ query positions per CTA (compile time: a position's partial results live in registers), DVL = ceil(dv / 32)
template <int DVL, int TQ>
__global__ void __launch_bounds__(TQ > 2 ? 512 : 1024, 1) talk_attention_kernel(SeqIndex ix, const int* cu_q, const int* seq_slot,
                                                                         const float* q, long long ldq, TalkDims d,
                                                                         const float* talk, const float* sink,
                                                                         PagedRows cache, void* out, int of32, long long ldo,
                                                                         float out_scale, TalkTile tl, float* part, int nsplit) {
    extern __shared__ __align__(16) float sm[];
    const int seq = blockIdx.y;
    const int t0 = cu_q[seq] + blockIdx.x * TQ, t1 = min(cu_q[seq + 1], t0 + TQ);
    if (t0 >= t1) return;
    const int nq = t1 - t0;
    const int H = d.heads, G = d.kv_heads, dk = d.dk, dv = d.dv, TK = tl.tk;
    const int lane = threadIdx.x & 31, h = threadIdx.x >> 5, nthr = blockDim.x;
    const int kvh = h / (H / G);
    const int slot = seq_slot[seq];
    const int pos0 = ix.positions[t0], pos1 = pos0 + nq - 1;   // a sequence's new tokens are consecutive positions
    float* qs = sm;                                   // [H][dk][TQ]
    float* Ks = qs + H * dk * TQ;                     // [TK][ks_stride]
    float* Vs = Ks + ((TK * tl.ks_stride + 3) & ~3);  // [TK][G * dv]
    float* Ss = Vs + ((TK * G * dv + 3) & ~3);        // [H][TQ][32] capped scores of every head
    float* Ps = Ss + H * TQ * 32;                     // [H][32][TQ] softmax weights, private to the head's warp
    float* Ts = Ps + H * 32 * TQ;                     // [H][H]
    for (int i = threadIdx.x; i < H * dk * TQ; i += nthr) {
        const int t = i % TQ, c = i / TQ;             // c = head * dk + coordinate
        float qv = t < nq ? q[(long long)(t0 + t) * ldq + c] : 0.f;
        // bf16 cache rows: the queries take the keys' precision, as in the tensor-core form, so that a position's
        // scores are the same products whichever kernel serves its step
        if (!cache.f32) qv = __bfloat162float(__float2bfloat16(qv));
        qs[i] = qv;
    }
    for (int i = threadIdx.x; i < H * H; i += nthr) Ts[i] = talk ? talk[i] : ((i / H) == (i % H) ? 1.f : 0.f);
    float mx[TQ], sum[TQ], O[TQ][DVL];
    const bool whole = nsplit <= 1;     // a share of the keys starts from nothing: the merge adds the sink once
#pragma unroll
    for (int t = 0; t < TQ; ++t) {
        mx[t] = sink && whole ? sink[h] : -INFINITY;
        sum[t] = sink && whole ? 1.f : 0.f;
#pragma unroll
        for (int i = 0; i < DVL; ++i) O[t][i] = 0.f;
    }
    const int lo_pos = max(0, pos0 - d.window + 1);
    const int nk = G * dk, nv = G * dv, row_elems = nk + nv;
    int kt_lo = lo_pos / TK, kt_hi = pos1 / TK;
    if (!whole) {       // this CTA's share of the key tiles
        const int per = (kt_hi - kt_lo + nsplit) / nsplit;
        kt_lo += blockIdx.z * per;
        kt_hi = min(kt_hi, kt_lo + per - 1);
    }
    for (int kt = kt_lo; kt <= kt_hi; ++kt) {
        const int j0 = kt * TK;
        __syncthreads();   // the previous tile is consumed (and, the first time, the queries are staged)
        if (tl.vec) {
            for (int t = h; t < TK; t += H) {
                const int j = j0 + t;
                const bool valid = j <= pos1;
                const long long row = valid ? cache_row(cache, slot, j) * row_elems : 0;
                if (cache.f32)
                    stage_row_vec(static_cast<const float*>(cache.pool) + row, valid, Ks + t * tl.ks_stride, Vs + t * nv, nk, nv, lane);
                else
                    stage_row_vec(static_cast<const __nv_bfloat16*>(cache.pool) + row, valid, Ks + t * tl.ks_stride, Vs + t * nv,
                                  nk, nv, lane);
            }
        } else {
            for (int i = threadIdx.x; i < TK * row_elems; i += nthr) {
                const int t = i / row_elems, c = i - t * row_elems;
                const int j = j0 + t;
                const float v = j <= pos1 ? ldx(cache.pool, cache_row(cache, slot, j) * row_elems + c, cache.f32) : 0.f;
                if (c < nk)
                    Ks[t * tl.ks_stride + c] = v;
                else
                    Vs[t * nv + c - nk] = v;
            }
        }
        __syncthreads();
        {   // scores of this warp's head for all TQ positions: lane = key, a key coordinate is read once for all of them
            float s[TQ];
#pragma unroll
            for (int t = 0; t < TQ; ++t) s[t] = 0.f;
            if (lane < TK) {
                const float* qh = qs + (long long)h * dk * TQ;
                const float* kp = Ks + lane * tl.ks_stride + kvh * dk;
#pragma unroll 4
                for (int c = 0; c < dk; ++c) {
                    const float kc = kp[c];
                    float qc[TQ];
                    load_tq<TQ>(qh + c * TQ, qc);
#pragma unroll
                    for (int t = 0; t < TQ; ++t) s[t] = fmaf(qc[t], kc, s[t]);
                }
            }
#pragma unroll
            for (int t = 0; t < TQ; ++t) {
                float v = s[t] * d.scale;
                if (d.softcap > 0.f) v = d.softcap * tanhf(v / d.softcap);
                Ss[(h * TQ + t) * 32 + lane] = v;
            }
        }
        __syncthreads();
#pragma unroll
        for (int t = 0; t < TQ; ++t) {
            const int pi = pos0 + t;
            float s = 0.f;
            for (int g = 0; g < H; ++g) s = fmaf(Ts[h * H + g], Ss[(g * TQ + t) * 32 + lane], s);
            const int j = j0 + lane;
            const bool ok = t < nq && lane < TK && j <= pi && pi - j < d.window;
            const float m_new = fmaxf(mx[t], warp_max(ok ? s : -INFINITY));
            const float p = ok ? expf(s - m_new) : 0.f;
            const float corr = mx[t] == -INFINITY ? 0.f : expf(mx[t] - m_new);   // a position that has seen nothing yet keeps zeros
            sum[t] = sum[t] * corr + warp_sum(p);
            mx[t] = m_new;
#pragma unroll
            for (int i = 0; i < DVL; ++i) O[t][i] *= corr;
            Ps[(h * 32 + lane) * TQ + t] = p;
        }
        __syncwarp();
        {   // values: lane = value column, a value is read once for all TQ positions
            const float* vb = Vs + kvh * dv + lane;
            const float* pb = Ps + (long long)h * 32 * TQ;
            for (int k = 0; k < TK; ++k) {
                float pk[TQ];
                load_tq<TQ>(pb + k * TQ, pk);
#pragma unroll
                for (int i = 0; i < DVL; ++i) {
                    if (lane + 32 * i < dv) {
                        const float vv = vb[k * nv + 32 * i];
#pragma unroll
                        for (int t = 0; t < TQ; ++t) O[t][i] = fmaf(pk[t], vv, O[t][i]);
                    }
                }
            }
        }
        __syncwarp();
    }
    if (!whole) {       // unnormalised sums, maximum and denominator of this share: [row][share][head][dv + 2]
#pragma unroll
        for (int t = 0; t < TQ; ++t) {
            if (t >= nq) continue;
            float* dst = part + (((long long)(t0 + t) * nsplit + blockIdx.z) * H + h) * (dv + 2);
#pragma unroll
            for (int i = 0; i < DVL; ++i)
                if (lane + 32 * i < dv) dst[lane + 32 * i] = O[t][i];
            if (lane == 0) dst[dv] = mx[t], dst[dv + 1] = sum[t];
        }
        return;
    }
#pragma unroll
    for (int t = 0; t < TQ; ++t) {
        if (t >= nq) continue;
        const float r = out_scale / sum[t];
#pragma unroll
        for (int i = 0; i < DVL; ++i)
            if (lane + 32 * i < dv) stx(out, (long long)(t0 + t) * ldo + (long long)h * dv + lane + 32 * i, of32, O[t][i] * r);
    }
}

// ---------------------------------------------------------------------------------------------- tensor-core form
// bf16 cache rows, 16 query positions per CTA, one warp per head, key tiles of 32 positions (multiples of 32, as above).
// Queries are rounded to bf16 once; keys and values arrive by cp.async in the cache's bf16 and are read through
// ldmatrix.  Per tile: S = Q K^T on mma.sync m16n8k16 (fp32 accumulation), scale and cap in registers, every head's
// scores to shared memory, barrier; the key buffer is free and the next tile's keys start to arrive while each warp
// mixes its head's scores (fp32, in the accumulator's own layout), updates the running softmax and multiplies the
// weights, as two bf16 terms (value + residual), with the values; barrier; the next tile's values start to arrive.
constexpr int TM_TK = 32, TM_TQ = 16, TM_SS = 40;   // key tile, query tile, floats per score row (32 + padding)

__device__ __forceinline__ void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// NDV = value size / 8.  PAIR: 17 to 32 heads run as a cluster of two CTAs with half of the heads each; a CTA computes
// its heads' scores and writes them into BOTH CTAs' shared memory (distributed shared memory), so that each can mix
// its heads' rows from all heads; two cluster barriers per tile take the place of two CTA barriers.  Both CTAs of a
// pair serve the same query tile, so they run the same number of tiles and meet at every barrier.
template <int NDV, bool PAIR>
__global__ void __launch_bounds__(512, 1) talk_attention_mma_kernel(SeqIndex ix, const int* cu_q, const int* seq_slot,
                                                                    const float* q, long long ldq, TalkDims d,
                                                                    const float* talk, const float* sink, PagedRows cache,
                                                                    void* out, int of32, long long ldo, float out_scale) {
    extern __shared__ __align__(16) unsigned char smraw[];
    const int seq = blockIdx.y;
    const int z = PAIR ? (int)(blockIdx.x & 1) : 0;                  // rank in the pair
    const int t0 = cu_q[seq] + (PAIR ? blockIdx.x >> 1 : blockIdx.x) * TM_TQ, t1 = min(cu_q[seq + 1], t0 + TM_TQ);
    if (t0 >= t1) return;                                            // the same for both CTAs of a pair
    const int nq = t1 - t0;
    const int H = d.heads, G = d.kv_heads, dk = d.dk;
    const int Hc = PAIR ? H / 2 : H;                                 // heads of this CTA: z * Hc ...
    constexpr int dv = NDV * 8;
    const int lane = threadIdx.x & 31, hl = threadIdx.x >> 5, nthr = blockDim.x;
    const int h = z * Hc + hl;                                       // this warp's head
    const int g_lo = (z * Hc) / (H / G), g_hi = (z * Hc + Hc - 1) / (H / G), Gc = g_hi - g_lo + 1;   // key/value heads staged
    const int kvh = h / (H / G) - g_lo;
    const int slot = seq_slot[seq];
    const int pos0 = ix.positions[t0], pos1 = pos0 + nq - 1;
    const int qstride = Hc * dk + 8, kstride = Gc * dk + 8, vstride = Gc * dv + 8;  // bf16 elements; rows 16 bytes apart mod 128
    // the scores come first: their place must be the same in both CTAs of a pair, whatever the other sizes
    float* Ss = reinterpret_cast<float*>(smraw);                                  // [H][16][TM_SS]
    float* Ts = Ss + H * TM_TQ * TM_SS;                                           // [Hc][H]
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(Ts + ((Hc * H + 3) & ~3));   // [16][qstride]
    __nv_bfloat16* Ks = Qs + TM_TQ * qstride;                                     // [32][kstride]
    __nv_bfloat16* Vs = Ks + TM_TK * kstride;                                     // [32][vstride]
    for (int i = threadIdx.x; i < TM_TQ * Hc * dk; i += nthr) {
        const int t = i / (Hc * dk), c = i - t * (Hc * dk);
        Qs[t * qstride + c] = __float2bfloat16(t < nq ? q[(long long)(t0 + t) * ldq + z * Hc * dk + c] : 0.f);
    }
    for (int i = threadIdx.x; i < Hc * H; i += nthr) {
        const int row = z * Hc + i / H, col = i % H;
        Ts[i] = talk ? talk[row * H + col] : (row == col ? 1.f : 0.f);
    }
    const int nk = G * dk, row_elems = nk + G * dv;
    const __nv_bfloat16* pool = static_cast<const __nv_bfloat16*>(cache.pool);
    const int kvec = Gc * dk / 8, vvec = Gc * dv / 8;
    const int koff = g_lo * dk, voff = nk + g_lo * dv;                 // this CTA's key / value heads within a cache row
    auto fetch_k = [&](int kt) {
        if (kt >= 0) {
            for (int i = threadIdx.x; i < TM_TK * kvec; i += nthr) {
                const int t = i / kvec, c = i - t * kvec;
                const int j = kt * TM_TK + t;
                const bool ok = j <= pos1;
                const __nv_bfloat16* src = pool + (ok ? cache_row(cache, slot, j) * row_elems + koff + c * 8 : 0);
                cp_async16((uint32_t)__cvta_generic_to_shared(Ks + t * kstride + c * 8), src, ok);
            }
        }
        cp_async_commit();
    };
    auto fetch_v = [&](int kt) {
        if (kt >= 0) {
            for (int i = threadIdx.x; i < TM_TK * vvec; i += nthr) {
                const int t = i / vvec, c = i - t * vvec;
                const int j = kt * TM_TK + t;
                const bool ok = j <= pos1;
                const __nv_bfloat16* src = pool + (ok ? cache_row(cache, slot, j) * row_elems + voff + c * 8 : 0);
                cp_async16((uint32_t)__cvta_generic_to_shared(Vs + t * vstride + c * 8), src, ok);
            }
        }
        cp_async_commit();
    };
    const int gq = lane >> 2, tq = lane & 3;          // accumulator rows gq and gq + 8, columns 8 n + 2 tq + {0, 1}
    float O[NDV][4];
#pragma unroll
    for (int n = 0; n < NDV; ++n) O[n][0] = O[n][1] = O[n][2] = O[n][3] = 0.f;
    const float m0 = sink ? sink[h] : -INFINITY;
    float mrow[2] = {m0, m0}, lrow[2] = {0.f, 0.f};
    const int kt_lo = max(0, pos0 - d.window + 1) / TM_TK, kt_hi = pos1 / TM_TK;
    fetch_k(kt_lo);
    fetch_v(kt_lo);
    const uint32_t q_addr = (uint32_t)__cvta_generic_to_shared(Qs + (lane & 15) * qstride + hl * dk + (lane >> 4) * 8);
    const uint32_t k_addr = (uint32_t)__cvta_generic_to_shared(Ks + ((lane & 7) + (lane >> 4) * 8) * kstride + kvh * dk + ((lane >> 3) & 1) * 8);
    const uint32_t v_addr = (uint32_t)__cvta_generic_to_shared(Vs + ((lane & 7) + ((lane >> 3) & 1) * 8) * vstride + kvh * dv + (lane >> 4) * 8);
    for (int kt = kt_lo; kt <= kt_hi; ++kt) {
        const int j0 = kt * TM_TK;
        cp_async_wait<1>();      // this tile's keys (its values may still be on their way)
        __syncthreads();
        float acc[4][4];
#pragma unroll
        for (int n = 0; n < 4; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
        for (int ks = 0; ks < dk; ks += 16) {
            uint32_t a[4], b[4];
            ldsm_x4(q_addr + ks * 2, a);
#pragma unroll
            for (int n2 = 0; n2 < 2; ++n2) {
                ldsm_x4(k_addr + (n2 * 16 * kstride + ks) * 2, b);
                mma_bf16(acc[2 * n2], a, b[0], b[1]);
                mma_bf16(acc[2 * n2 + 1], a, b[2], b[3]);
            }
        }
        float* sh = Ss + (h * TM_TQ) * TM_SS;
        uint32_t peer = 0;
        if constexpr (PAIR) {
            const uint32_t mine = (uint32_t)__cvta_generic_to_shared(sh);
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(peer) : "r"(mine), "r"(z ^ 1));
        }
#pragma unroll
        for (int n = 0; n < 4; ++n) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float v = acc[n][i] * d.scale;
                if (d.softcap > 0.f) v = d.softcap * tanhf(v / d.softcap);
                acc[n][i] = v;
            }
            const int o0 = gq * TM_SS + 8 * n + 2 * tq, o1 = (gq + 8) * TM_SS + 8 * n + 2 * tq;
            *reinterpret_cast<float2*>(sh + o0) = make_float2(acc[n][0], acc[n][1]);
            *reinterpret_cast<float2*>(sh + o1) = make_float2(acc[n][2], acc[n][3]);
            if constexpr (PAIR) {      // the same rows of the other CTA's copy
                asm volatile("st.shared::cluster.v2.f32 [%0], {%1, %2};" ::"r"(peer + o0 * 4), "f"(acc[n][0]), "f"(acc[n][1]) : "memory");
                asm volatile("st.shared::cluster.v2.f32 [%0], {%1, %2};" ::"r"(peer + o1 * 4), "f"(acc[n][2]), "f"(acc[n][3]) : "memory");
            }
        }
        if constexpr (PAIR)
            cluster_barrier();   // every head's scores are in both CTAs; the key buffer is free
        else
            __syncthreads();     // every head's scores are there; the key buffer is free
        fetch_k(kt < kt_hi ? kt + 1 : -1);
#pragma unroll
        for (int n = 0; n < 4; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
        for (int g = 0; g < H; ++g) {
            const float w = Ts[hl * H + g];
            const float* sg = Ss + (g * TM_TQ) * TM_SS + 2 * tq;
#pragma unroll
            for (int n = 0; n < 4; ++n) {
                const float2 lo = *reinterpret_cast<const float2*>(sg + gq * TM_SS + 8 * n);
                const float2 hi = *reinterpret_cast<const float2*>(sg + (gq + 8) * TM_SS + 8 * n);
                acc[n][0] = fmaf(w, lo.x, acc[n][0]);
                acc[n][1] = fmaf(w, lo.y, acc[n][1]);
                acc[n][2] = fmaf(w, hi.x, acc[n][2]);
                acc[n][3] = fmaf(w, hi.y, acc[n][3]);
            }
        }
        // mask, running maximum and weights of rows gq (r = 0) and gq + 8 (r = 1)
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int row = gq + 8 * r, pi = pos0 + row;
            float tmax = -INFINITY;
#pragma unroll
            for (int n = 0; n < 4; ++n)
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const int j = j0 + 8 * n + 2 * tq + c;
                    const bool ok = row < nq && j <= pi && pi - j < d.window;
                    if (!ok) acc[n][2 * r + c] = -INFINITY;
                    tmax = fmaxf(tmax, acc[n][2 * r + c]);
                }
            tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
            tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
            const float m_new = fmaxf(mrow[r], tmax);
            const float corr = mrow[r] == -INFINITY ? 0.f : expf(mrow[r] - m_new);
            float part = 0.f;
#pragma unroll
            for (int n = 0; n < 4; ++n)
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const float sv = acc[n][2 * r + c];
                    const float p = sv == -INFINITY ? 0.f : expf(sv - m_new);
                    acc[n][2 * r + c] = p;
                    part += p;
                }
            lrow[r] = lrow[r] * corr + part;
            mrow[r] = m_new;
#pragma unroll
            for (int n = 0; n < NDV; ++n) {
                O[n][2 * r] *= corr;
                O[n][2 * r + 1] *= corr;
            }
        }
        cp_async_wait<1>();      // this tile's values
        __syncthreads();
#pragma unroll
        for (int j = 0; j < 2; ++j) {        // 16 keys per step
            uint32_t ph[4], pl[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float x0 = acc[2 * j + (i >> 1)][2 * (i & 1)], x1 = acc[2 * j + (i >> 1)][2 * (i & 1) + 1];
                const __nv_bfloat16 h0 = __float2bfloat16(x0), h1 = __float2bfloat16(x1);
                __nv_bfloat162 hv;
                hv.x = h0, hv.y = h1;
                ph[i] = *reinterpret_cast<uint32_t*>(&hv);
                pl[i] = pack_bf16(x0 - __bfloat162float(h0), x1 - __bfloat162float(h1));
            }
#pragma unroll
            for (int n = 0; n < NDV; n += 2) {
                uint32_t b[4];
                ldsm_x4_t(v_addr + (j * 16 * vstride + n * 8) * 2, b);
                mma_bf16(O[n], ph, b[0], b[1]);
                mma_bf16(O[n], pl, b[0], b[1]);
                mma_bf16(O[n + 1], ph, b[2], b[3]);
                mma_bf16(O[n + 1], pl, b[2], b[3]);
            }
        }
        if constexpr (PAIR)
            cluster_barrier();   // the value buffer is free, and the other CTA is done reading this tile's scores
        else
            __syncthreads();     // the value buffer is free
        fetch_v(kt < kt_hi ? kt + 1 : -1);
    }
    cp_async_wait<0>();
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = gq + 8 * r;
        float l = lrow[r];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        if (sink) l += expf(sink[h] - mrow[r]);
        if (row >= nq) continue;
        const float sc = out_scale / l;
#pragma unroll
        for (int n = 0; n < NDV; ++n) {
            const long long o = (long long)(t0 + row) * ldo + (long long)h * dv + 8 * n + 2 * tq;
            stx(out, o, of32, O[n][2 * r] * sc);
            stx(out, o + 1, of32, O[n][2 * r + 1] * sc);
        }
    }
}

// one warp per (token, head): the shares' sums brought to a common maximum, the sink entering once.  lane = share (at
// most 32).  `fresh`: the partial results were written by other CTAs of the SAME launch (read past the L1 cache).
template <bool FRESH>
__device__ __forceinline__ void merge_shares(const float* base, long long step, int nsplit, const float* sink, int h, void* out,
                                             int of32, long long orow, float out_scale, int dv, int lane) {
    auto ld = [](const float* p) { return FRESH ? __ldcg(p) : __ldg(p); };
    const float ms = lane < nsplit ? ld(base + lane * step + dv) : -INFINITY;
    const float ls = lane < nsplit ? ld(base + lane * step + dv + 1) : 0.f;
    const float top = fmaxf(sink ? sink[h] : -INFINITY, warp_max(ms));
    const float ws = ms == -INFINITY ? 0.f : expf(ms - top);
    const float den = warp_sum(ls * ws) + (sink ? expf(sink[h] - top) : 0.f);
    const float r = out_scale / den;
    for (int c0 = 0; c0 < dv; c0 += 32) {
        const int c = c0 + lane;
        float o = 0.f;
#pragma unroll 8
        for (int s = 0; s < nsplit; ++s) {
            const float w = __shfl_sync(0xffffffffu, ws, s);
            o = fmaf(c < dv ? ld(base + s * step + c) : 0.f, w, o);
        }
        if (c < dv) stx(out, orow + c, of32, o * r);
    }
}

__global__ void talk_merge_kernel(const float* part, int nsplit, const float* sink, void* out, int of32, long long ldo,
                                  float out_scale, int M, int H, int dv) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long idx = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
    if (idx >= (long long)M * H) return;
    const int m = (int)(idx / H), h = (int)(idx - (long long)m * H);
    merge_shares<false>(part + ((long long)m * nsplit * H + h) * (dv + 2), (long long)H * (dv + 2), nsplit, sink, h, out, of32,
                        (long long)m * ldo + (long long)h * dv, out_scale, dv, lane);
}

// ---------------------------------------------------------------------------------------------- steps of few tokens
// One CTA per (token, share of its key tiles), one warp per head, nothing staged: lane = key reads its own cache row in
// 16-byte pieces (several in flight) against the query in shared memory; the capped scores go to shared memory (two
// buffers, one barrier per tile); every warp mixes its head's row, updates the running softmax and adds the values with
// each lane on four neighbouring value columns, the rows' addresses passed from lane to lane.  Small shared memory and
// few registers: several CTAs share an SM and hide one another's loads.
// DPL > 0 (key size = 8 DPL): eight lanes share a key row, DPL coordinates each, against query coordinates held in
// registers, so that a row is read in whole 128-byte lines; four keys per step, sums closed by shuffles.  DPL = 0 (any
// key size that is a multiple of the 16-byte piece): lane = key reads its own row.
template <typename T, int DPL>
__global__ void __launch_bounds__(1024, 1) talk_decode_kernel(SeqIndex ix, const float* q, long long ldq, TalkDims d,
                                                              const float* talk, const float* sink, PagedRows cache, void* out,
                                                              int of32, long long ldo, float out_scale, float* part, int nsplit,
                                                              int* arrived) {
    constexpr int VE = 16 / sizeof(T);
    extern __shared__ __align__(16) float sm[];
    const int m = blockIdx.x;
    const int H = d.heads, G = d.kv_heads, dk = d.dk, dv = d.dv;
    const int lane = threadIdx.x & 31, h = threadIdx.x >> 5, nthr = blockDim.x;
    const int kvh = h / (H / G);
    const int slot = ix.token_slot[m], pos = ix.positions[m];
    float* qs = sm;                        // [H][dk]
    float* Ss = qs + ((H * dk + 3) & ~3);  // [2][H][32]
    float* Ps = Ss + 2 * H * 32;           // [H][32]
    float* Ts = Ps + H * 32;               // [H][H]
    for (int i = threadIdx.x; i < H * dk; i += nthr) {
        float qv = q[(long long)m * ldq + i];
        if (sizeof(T) == 2) qv = __bfloat162float(__float2bfloat16(qv));
        qs[i] = qv;
    }
    for (int i = threadIdx.x; i < H * H; i += nthr) Ts[i] = talk ? talk[i] : ((i / H) == (i % H) ? 1.f : 0.f);
    const bool whole = nsplit <= 1;
    float mx = sink && whole ? sink[h] : -INFINITY, sum = sink && whole ? 1.f : 0.f;
    float O[2][4];
#pragma unroll
    for (int a = 0; a < 2; ++a) O[a][0] = O[a][1] = O[a][2] = O[a][3] = 0.f;
    const int lo_pos = max(0, pos - d.window + 1);
    int kt_lo = lo_pos / 32, kt_hi = pos / 32;
    if (!whole) {
        const int per = (kt_hi - kt_lo + nsplit) / nsplit;
        kt_lo += blockIdx.y * per;
        kt_hi = min(kt_hi, kt_lo + per - 1);
    }
    const int nk = G * dk, row_elems = nk + G * dv;
    const T* pool = static_cast<const T*>(cache.pool);
    const float* qh = qs + h * dk;
    const int groups = dv >> 2;            // four value columns per lane and group
    __syncthreads();
    float qreg[DPL > 0 ? DPL : 1];
    if constexpr (DPL > 0) {
#pragma unroll
        for (int i = 0; i < DPL; ++i) qreg[i] = qh[(lane & 7) * DPL + i];
    }
    int par = 0;
    // a tile's row addresses are looked up one tile ahead, and lines that are needed later are asked for early: this
    // tile's value rows before its key rows are read, the next tile's key rows behind them
    auto row_of = [&](int kt) {
        const int j = kt * 32 + lane;
        return kt <= kt_hi && j >= lo_pos && j <= pos ? cache_row(cache, slot, j) * row_elems : -1;
    };
    auto ask = [&](const T* p, int elems) {
        for (int e = 0; e < elems; e += 128 / (int)sizeof(T)) asm volatile("prefetch.global.L1 [%0];" ::"l"(p + e));
    };
    long long row_next = row_of(kt_lo);
    for (int kt = kt_lo; kt <= kt_hi; ++kt, par ^= 1) {
        const bool ok = row_next >= 0;
        const long long row = ok ? row_next : 0;
        row_next = row_of(kt + 1);
        float s = 0.f;
        if (ok) ask(pool + row + nk + kvh * dv, dv);
        if constexpr (DPL > 0) {
            const int sub = lane & 7, kg = lane >> 3;
#pragma unroll
            for (int it = 0; it < 8; ++it) {
                const long long rk = __shfl_sync(0xffffffffu, row, 4 * it + kg);      // a masked key reads row 0 of the pool
                const uint4* kp = reinterpret_cast<const uint4*>(pool + rk + kvh * dk + sub * DPL);
                uint4 r[DPL / VE];
#pragma unroll
                for (int u = 0; u < DPL / VE; ++u) r[u] = __ldg(kp + u);
                float s0 = 0.f, s1 = 0.f;
#pragma unroll
                for (int u = 0; u < DPL / VE; ++u) {
                    const T* x = reinterpret_cast<const T*>(&r[u]);
#pragma unroll
                    for (int i = 0; i < VE; i += 2) {
                        s0 = fmaf(qreg[u * VE + i], (float)x[i], s0);
                        s1 = fmaf(qreg[u * VE + i + 1], (float)x[i + 1], s1);
                    }
                }
                float t = s0 + s1;
                t += __shfl_xor_sync(0xffffffffu, t, 1);
                t += __shfl_xor_sync(0xffffffffu, t, 2);
                t += __shfl_xor_sync(0xffffffffu, t, 4);
                const float mine = __shfl_sync(0xffffffffu, t, (lane & 3) * 8);     // key 4 it + (lane & 3)
                if ((lane >> 2) == it) s = mine;
            }
            s *= d.scale;
            if (d.softcap > 0.f) s = d.softcap * tanhf(s / d.softcap);
        } else if (ok) {
            const uint4* kp = reinterpret_cast<const uint4*>(pool + row + kvh * dk);
            float s0 = 0.f, s1 = 0.f;
            for (int c0 = 0; c0 < dk; c0 += 8 * VE) {
                uint4 r[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) r[u] = c0 + u * VE < dk ? __ldg(kp + c0 / VE + u) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    if (c0 + u * VE >= dk) continue;
                    const T* x = reinterpret_cast<const T*>(&r[u]);
                    const float* qc = qh + c0 + u * VE;
#pragma unroll
                    for (int i = 0; i < VE; i += 2) {
                        s0 = fmaf(qc[i], (float)x[i], s0);
                        s1 = fmaf(qc[i + 1], (float)x[i + 1], s1);
                    }
                }
            }
            s = (s0 + s1) * d.scale;
            if (d.softcap > 0.f) s = d.softcap * tanhf(s / d.softcap);
        }
        if (row_next >= 0) ask(pool + row_next + kvh * dk, dk);
        float* sb = Ss + par * H * 32;
        sb[h * 32 + lane] = s;
        __syncthreads();
        float mixed = 0.f;
        for (int g = 0; g < H; ++g) mixed = fmaf(Ts[h * H + g], sb[g * 32 + lane], mixed);
        const float m_new = fmaxf(mx, warp_max(ok ? mixed : -INFINITY));
        const float p = ok ? expf(mixed - m_new) : 0.f;
        const float corr = mx == -INFINITY ? 0.f : expf(mx - m_new);
        sum = sum * corr + warp_sum(p);
        mx = m_new;
#pragma unroll
        for (int a = 0; a < 2; ++a) O[a][0] *= corr, O[a][1] *= corr, O[a][2] *= corr, O[a][3] *= corr;
        const long long vrow = row + nk + kvh * dv;
        // no branch on a zero weight: the loads of eight keys stay in flight together (a masked key's row is row 0 of
        // the pool, readable and multiplied by zero)
#pragma unroll 8
        for (int k = 0; k < 32; ++k) {
            const float pk = __shfl_sync(0xffffffffu, p, k);
            const long long vr = __shfl_sync(0xffffffffu, vrow, k);
#pragma unroll
            for (int a = 0; a < 2; ++a) {
                const int gi = lane + 32 * a;
                if (gi < groups) {
                    float v0, v1, v2, v3;
                    if (sizeof(T) == 2) {
                        const uint2 raw = __ldg(reinterpret_cast<const uint2*>(pool + vr + 4 * gi));
                        const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
                        const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
                        v0 = __bfloat162float(lo.x), v1 = __bfloat162float(lo.y), v2 = __bfloat162float(hi.x), v3 = __bfloat162float(hi.y);
                    } else {
                        const float4 raw = __ldg(reinterpret_cast<const float4*>(pool + vr + 4 * gi));
                        v0 = raw.x, v1 = raw.y, v2 = raw.z, v3 = raw.w;
                    }
                    O[a][0] = fmaf(pk, v0, O[a][0]);
                    O[a][1] = fmaf(pk, v1, O[a][1]);
                    O[a][2] = fmaf(pk, v2, O[a][2]);
                    O[a][3] = fmaf(pk, v3, O[a][3]);
                }
            }
        }
    }
    if (!whole) {
        float* dst = part + (((long long)m * nsplit + blockIdx.y) * H + h) * (dv + 2);
#pragma unroll
        for (int a = 0; a < 2; ++a)
            if (lane + 32 * a < groups)
#pragma unroll
                for (int i = 0; i < 4; ++i) dst[4 * (lane + 32 * a) + i] = O[a][i];
        if (lane == 0) dst[dv] = mx, dst[dv + 1] = sum;
        if (!arrived) return;       // a kernel of its own merges
        // the token's last CTA to arrive merges its shares (one launch less); it puts the counter back for the next step
        __shared__ int last;
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) {
            const int t = atomicAdd(arrived + m, 1);
            last = t == nsplit - 1;
            if (last) arrived[m] = 0;
        }
        __syncthreads();
        if (!last) return;
        __threadfence();
        merge_shares<true>(part + ((long long)m * nsplit * H + h) * (dv + 2), (long long)H * (dv + 2), nsplit, sink, h, out, of32,
                           (long long)m * ldo + (long long)h * dv, out_scale, dv, lane);
        return;
    }
    const float r = out_scale / sum;
#pragma unroll
    for (int a = 0; a < 2; ++a)
        if (lane + 32 * a < groups)
#pragma unroll
            for (int i = 0; i < 4; ++i)
                stx(out, (long long)m * ldo + (long long)h * dv + 4 * (lane + 32 * a) + i, of32, O[a][i] * r);
}

}  // namespace

int launch_talk_post(const SeqIndex& ix, float* qkv, long long ld, const TalkDims& d, const float* bias, const float* q_norm,
                     const float* k_norm, float eps, const float* freq, const PagedRows& cache, cudaStream_t stream) {
    if (ix.M <= 0) return 0;
    if (d.rot_dims > 0 && !freq) return set_error("talk_post: no rotation frequencies");
    const long long warps = (long long)ix.M * (d.heads + 2 * d.kv_heads);
    talk_post_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, stream>>>(ix, qkv, ld, d, bias, q_norm, k_norm, eps, freq, cache);
    count_launch(1);
    ASD_CUDA(cudaGetLastError());
    return 0;
}

int launch_talk_attention(const SeqIndex& ix, const int* cu_q, const int* seq_slot, int nseq, int max_qlen, int max_kv_len,
                          const float* q, long long ldq, const TalkDims& d, const float* talk, const float* sink,
                          const PagedRows& cache, void* out, int of32, long long ldo, float out_scale, const AttnSplit& ws,
                          cudaStream_t stream) {
    if (ix.M <= 0 || nseq <= 0) return 0;
    if (d.heads <= 0 || d.heads > 32 || d.kv_heads <= 0 || d.heads % d.kv_heads)
        return set_error("talk_attention: %d heads (at most 32) over %d key/value heads", d.heads, d.kv_heads);
    if (d.dv > 256 || d.dv <= 0 || d.dk <= 0 || d.window <= 0) return set_error("talk_attention: bad sizes");
    // bf16 cache rows and sizes that fill the tensor-core fragments: prompts and portions take the mma.sync kernel, up to
    // 16 heads in one CTA, 17 to 32 (an even number) in a cluster of two
    if (ws.tiled && !cache.f32 && max_qlen >= 8 && d.heads <= 32 && (d.heads <= 16 || d.heads % 2 == 0) && d.dk % 16 == 0 &&
        (d.dv == 16 || d.dv == 32 || d.dv == 64 || d.dv == 128) && (reinterpret_cast<uintptr_t>(cache.pool) & 15) == 0) {
        const bool pair = d.heads > 16;
        const int hc = pair ? d.heads / 2 : d.heads, per = d.heads / d.kv_heads;
        const int gc = pair ? (hc - 1) / per + 1 + ((hc % per) ? 1 : 0) : d.kv_heads;     // key/value heads a CTA stages at most
        const int gcc = gc < d.kv_heads ? gc : d.kv_heads;
        const size_t smem = (size_t)(TM_TQ * (hc * d.dk + 8) + TM_TK * (gcc * d.dk + 8) + TM_TK * (gcc * d.dv + 8)) * 2 +
                            (size_t)(d.heads * TM_TQ * TM_SS + ((hc * d.heads + 3) & ~3)) * sizeof(float);
        if (smem <= 220 * 1024) {
            const unsigned qtiles = (max_qlen + TM_TQ - 1) / TM_TQ;
            dim3 grid(pair ? 2 * qtiles : qtiles, nseq);
            if (grid.y > 65535) return set_error("talk_attention: too many sequences");
            cudaLaunchConfig_t lc = {};
            lc.gridDim = grid, lc.blockDim = dim3(hc * 32), lc.dynamicSmemBytes = smem, lc.stream = stream;
            cudaLaunchAttribute at[1];
            at[0].id = cudaLaunchAttributeClusterDimension;
            at[0].val.clusterDim.x = pair ? 2 : 1, at[0].val.clusterDim.y = 1, at[0].val.clusterDim.z = 1;
            lc.attrs = at, lc.numAttrs = 1;
#define ASD_TM_CASE2(N, P)                                                                                            \
    {                                                                                                                 \
        auto fn = talk_attention_mma_kernel<N, P>;                                                                    \
        static PerDeviceOnce once;                                                                                    \
        if (once.need()) ASD_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024)); \
        ASD_CUDA(cudaLaunchKernelEx(&lc, fn, ix, cu_q, seq_slot, q, ldq, d, talk, sink, cache, out, of32, ldo, out_scale)); \
    }
#define ASD_TM_CASE(N)                  \
    if (pair) ASD_TM_CASE2(N, true)     \
    else ASD_TM_CASE2(N, false)
            if (d.dv == 16) {
                ASD_TM_CASE(2)
            } else if (d.dv == 32) {
                ASD_TM_CASE(4)
            } else if (d.dv == 64) {
                ASD_TM_CASE(8)
            } else {
                ASD_TM_CASE(16)
            }
#undef ASD_TM_CASE
#undef ASD_TM_CASE2
            count_launch(1);
            ASD_CUDA(cudaGetLastError());
            return 0;
        }
    }
    // steps of few tokens: a CTA per (token, share of its key tiles), rows read straight from the cache
    {
        const int ve = cache.f32 ? 4 : 8;
        if (ws.tiled && max_qlen < 8 && d.dk % ve == 0 && d.dv % 4 == 0 && (d.kv_heads * d.dv) % ve == 0 &&
            (reinterpret_cast<uintptr_t>(cache.pool) & 15) == 0) {
            const int tiles = (int)((long long)(d.window < max_kv_len ? d.window : max_kv_len) + 31) / 32 + 1;
            int nsplit = 1;
            if (ws.o && tiles >= 4) {
                nsplit = (int)((148 * 4 + ix.M - 1) / ix.M);
                if (nsplit > tiles / 2) nsplit = tiles / 2;
                if (nsplit > 32) nsplit = 32;
                const long long per_share = (long long)ix.M * d.heads * (d.dv + 2);
                if ((long long)nsplit * per_share > ws.o_elems) nsplit = (int)(ws.o_elems / per_share);
                if (nsplit < 2) nsplit = 1;
            }
            const size_t smem = (size_t)(((d.heads * d.dk + 3) & ~3) + 3 * d.heads * 32 + d.heads * d.heads) * sizeof(float);
            dim3 grid(ix.M, nsplit);
            if (smem <= 48 * 1024 && nsplit <= 65535) {     // (the default limit of dynamic shared memory: no attribute to set)
                int* arrived = ws.ml && ws.rows >= ix.M ? reinterpret_cast<int*>(ws.ml) : nullptr;   // zeroed counters, one per token
                const int dpl = (d.dk % 8 == 0 && (d.dk / 8) % ve == 0 && d.dk / 8 <= 32) ? d.dk / 8 : 0;
#define ASD_TD_CASE(T_, D_)                                                                                            \
    {                                                                                                                 \
        auto fn = talk_decode_kernel<T_, D_>;                                                                         \
        fn<<<grid, d.heads * 32, smem, stream>>>(ix, q, ldq, d, talk, sink, cache, out, of32, ldo, out_scale, ws.o,    \
                                                 nsplit, arrived);                                                    \
    }
                if (cache.f32) {
                    if (dpl == 4) ASD_TD_CASE(float, 4)
                    else if (dpl == 8) ASD_TD_CASE(float, 8)
                    else if (dpl == 16) ASD_TD_CASE(float, 16)
                    else if (dpl == 32) ASD_TD_CASE(float, 32)
                    else ASD_TD_CASE(float, 0)
                } else {
                    if (dpl == 8) ASD_TD_CASE(__nv_bfloat16, 8)
                    else if (dpl == 16) ASD_TD_CASE(__nv_bfloat16, 16)
                    else if (dpl == 32) ASD_TD_CASE(__nv_bfloat16, 32)
                    else ASD_TD_CASE(__nv_bfloat16, 0)
                }
#undef ASD_TD_CASE
                count_launch(1);
                if (nsplit > 1 && !arrived) {
                    const long long warps = (long long)ix.M * d.heads;
                    talk_merge_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, stream>>>(ws.o, nsplit, sink, out, of32, ldo, out_scale,
                                                                                     ix.M, d.heads, d.dv);
                    count_launch(1);
                }
                ASD_CUDA(cudaGetLastError());
                return 0;
            }
        }
    }
    // Key tile and query tile from the layer's sizes (the key tile never depends on the batch: a position's sums run over
    // the same tiles whatever it is fed with); single-token steps take one query position per CTA.
    const int esz = cache.f32 ? 4 : 2, ve = 16 / esz;
    const int ks = (d.kv_heads * d.dk) | 1;
    auto need = [&](int tq, int tk) {
        return ((size_t)tq * d.heads * d.dk + (((size_t)tk * ks + 3) & ~(size_t)3) + (((size_t)tk * d.kv_heads * d.dv + 3) & ~(size_t)3) +
                2 * (size_t)tq * d.heads * 32 + (size_t)d.heads * d.heads) * sizeof(float);
    };
    int tk = 32;
    while (tk > 1 && need(1, tk) > 200 * 1024) tk >>= 1;
    if (need(1, tk) > 200 * 1024) return set_error("talk_attention: the heads' rows do not fit shared memory");
    int tq = d.heads > 16 ? 2 : 8;
    while (tq > 1 && (need(tq, tk) > 200 * 1024 || tq >= 2 * max_qlen)) tq >>= 1;
    TalkTile tl{tk, ks, 0};
    tl.vec = (d.kv_heads * d.dk) % ve == 0 && (d.kv_heads * d.dv) % ve == 0 && (reinterpret_cast<uintptr_t>(cache.pool) & 15) == 0;
    const size_t smem = need(tq, tk);
    dim3 grid((max_qlen + tq - 1) / tq, nseq);
    if (grid.y > 65535) return set_error("talk_attention: too many sequences");
    // few CTAs and many key tiles (single-token steps of a few sequences): the key tiles are cut into shares for several
    // CTAs, whose partial sums a second kernel merges
    int nsplit = 1;
    const long long ctas = (long long)grid.x * grid.y;
    const int tiles = (int)((long long)(d.window < max_kv_len ? d.window : max_kv_len) + tq) / tk + 1;
    if (ws.o && ctas * 2 <= 148 && tiles >= 4) {
        nsplit = (int)(148 / ctas);
        if (nsplit > tiles / 2) nsplit = tiles / 2;
        if (nsplit > 32) nsplit = 32;
        const long long per_share = (long long)ix.M * d.heads * (d.dv + 2);
        if ((long long)nsplit * per_share > ws.o_elems) nsplit = (int)(ws.o_elems / per_share);
        if (nsplit < 2) nsplit = 1;
    }
    grid.z = nsplit;
    const int dvl = (d.dv + 31) / 32;
#define ASD_TA_CASE2(L, Q)                                                                                            \
    {                                                                                                                 \
        auto fn = talk_attention_kernel<L, Q>;                                                                        \
        static PerDeviceOnce once;                                                                                    \
        if (once.need()) ASD_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024)); \
        fn<<<grid, d.heads * 32, smem, stream>>>(ix, cu_q, seq_slot, q, ldq, d, talk, sink, cache, out, of32, ldo,     \
                                                 out_scale, tl, ws.o, nsplit);                                        \
    }
#define ASD_TA_CASE(L)                      \
    if (tq == 8) ASD_TA_CASE2(L, 8)         \
    else if (tq == 4) ASD_TA_CASE2(L, 4)    \
    else if (tq == 2) ASD_TA_CASE2(L, 2)    \
    else ASD_TA_CASE2(L, 1)
    if (dvl <= 1) {
        ASD_TA_CASE(1)
    } else if (dvl <= 2) {
        ASD_TA_CASE(2)
    } else if (dvl <= 4) {
        ASD_TA_CASE(4)
    } else {
        ASD_TA_CASE(8)
    }
#undef ASD_TA_CASE
#undef ASD_TA_CASE2
    if (nsplit > 1) {
        const long long warps = (long long)ix.M * d.heads;
        talk_merge_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, stream>>>(ws.o, nsplit, sink, out, of32, ldo, out_scale, ix.M,
                                                                         d.heads, d.dv);
        count_launch(1);
    }
    count_launch(1);
    ASD_CUDA(cudaGetLastError());
    return 0;
}

}  // namespace asd
