// Talking-heads window attention: grouped-query softmax attention over a sliding window whose scores pass a tanh cap and
// are then mixed across the heads (s'_h = sum_g talk[h][g] s_g) before a softmax with a sink per head in its denominator.
// The mix needs every head's score of a (query, key) pair, so one CTA serves ALL heads of a tile of query positions.
// talk_post_kernel:  biases, RMS norm of every query / key head (plain weight), rotation of the leading coordinates in
//   pairs (2 i, 2 i + 1), queries left in place, keys and values appended to the paged cache; one warp per (token, head).
// talk_attention_kernel: one CTA per (sequence, TQ consecutive new positions), one warp per head.  Keys are visited in
//   tiles of TK positions that start at multiples of TK (a position's sums run over the same tiles in the same order
//   however its sequence was cut into forwards): the tile's keys and values are staged in shared memory as fp32 once
//   for all heads and all TQ queries; lane = key for the scores (capped, stored for the other heads), then every warp
//   mixes its head's row, folds it into the running softmax (which starts from the sink: maximum = sink, sum = 1,
//   nothing accumulated) and adds the values with lane = value column.
#include <cuda_bf16.h>
#include <math.h>

#include "asd_internal.h"
#include "blocks.h"
#include "elem.cuh"

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

// query positions per CTA at most: eight for up to 16 heads (512 threads, 128 registers each), two beyond

struct TalkTile {
    int tq, tk;            // query positions per CTA, key positions per tile (<= 32)
    int ks_stride;         // floats per staged key row (odd: lanes = keys read without bank conflicts)
};

template <int DVL, int TA_TQ>
__global__ void __launch_bounds__(TA_TQ > 2 ? 512 : 1024, 1) talk_attention_kernel(SeqIndex ix, const int* cu_q, const int* seq_slot,
                                                                 const float* q, long long ldq, TalkDims d, const float* talk,
                                                                 const float* sink, PagedRows cache, void* out, int of32,
                                                                 long long ldo, float out_scale, TalkTile tl) {
    extern __shared__ __align__(16) float sm[];
    const int seq = blockIdx.y;
    const int t0 = cu_q[seq] + blockIdx.x * tl.tq, t1 = min(cu_q[seq + 1], t0 + tl.tq);
    if (t0 >= t1) return;
    const int nq = t1 - t0;
    const int H = d.heads, G = d.kv_heads, dk = d.dk, dv = d.dv, TK = tl.tk;
    const int lane = threadIdx.x & 31, h = threadIdx.x >> 5, nthr = blockDim.x;
    const int kvh = h / (H / G);
    const int slot = seq_slot[seq];
    const int pos0 = ix.positions[t0], pos1 = pos0 + nq - 1;   // a sequence's new tokens are consecutive positions
    float* qs = sm;                                   // [tq][H][dk]
    float* Ks = qs + tl.tq * H * dk;                  // [TK][ks_stride]
    float* Vs = Ks + TK * tl.ks_stride;               // [TK][G * dv]
    float* Ss = Vs + TK * G * dv;                     // [tq][H][32]
    float* Ts = Ss + tl.tq * H * 32;                  // [H][H]
    for (int i = threadIdx.x; i < nq * H * dk; i += nthr) {
        const int t = i / (H * dk), c = i - t * (H * dk);
        qs[i] = q[(long long)(t0 + t) * ldq + c];
    }
    for (int i = threadIdx.x; i < H * H; i += nthr) Ts[i] = talk ? talk[i] : ((i / H) == (i % H) ? 1.f : 0.f);
    float mx[TA_TQ], sum[TA_TQ], O[TA_TQ][DVL];
#pragma unroll
    for (int t = 0; t < TA_TQ; ++t) {
        mx[t] = sink ? sink[h] : -INFINITY;
        sum[t] = sink ? 1.f : 0.f;
#pragma unroll
        for (int i = 0; i < DVL; ++i) O[t][i] = 0.f;
    }
    const int lo_pos = max(0, pos0 - d.window + 1);
    const int row_elems = G * (dk + dv);
    for (int kt = lo_pos / TK; kt <= pos1 / TK; ++kt) {
        const int j0 = kt * TK;
        __syncthreads();   // the previous tile is consumed (and, the first time, the queries are staged)
        for (int i = threadIdx.x; i < TK * G * dk; i += nthr) {
            const int t = i / (G * dk), c = i - t * (G * dk);
            const int j = j0 + t;
            Ks[t * tl.ks_stride + c] = j <= pos1 ? ldx(cache.pool, cache_row(cache, slot, j) * row_elems + c, cache.f32) : 0.f;
        }
        for (int i = threadIdx.x; i < TK * G * dv; i += nthr) {
            const int t = i / (G * dv), c = i - t * (G * dv);
            const int j = j0 + t;
            Vs[i] = j <= pos1 ? ldx(cache.pool, cache_row(cache, slot, j) * row_elems + (long long)G * dk + c, cache.f32) : 0.f;
        }
        __syncthreads();
        // scores of this warp's head: lane = key
#pragma unroll
        for (int t = 0; t < TA_TQ; ++t) {
            if (t >= nq) break;
            const int pi = pos0 + t;
            if (j0 > pi || j0 + TK - 1 < pi - d.window + 1) continue;   // no key of the tile is visible
            float s = 0.f;
            if (lane < TK) {
                const float* qv = qs + (t * H + h) * dk;
                const float* kv = Ks + lane * tl.ks_stride + kvh * dk;
                float s0 = 0.f, s1 = 0.f;
                int c = 0;
                for (; c + 1 < dk; c += 2) {
                    s0 = fmaf(qv[c], kv[c], s0);
                    s1 = fmaf(qv[c + 1], kv[c + 1], s1);
                }
                if (c < dk) s0 = fmaf(qv[c], kv[c], s0);
                s = (s0 + s1) * d.scale;
                if (d.softcap > 0.f) s = d.softcap * tanhf(s / d.softcap);
            }
            Ss[(t * H + h) * 32 + lane] = s;
        }
        __syncthreads();
#pragma unroll
        for (int t = 0; t < TA_TQ; ++t) {
            if (t >= nq) break;
            const int pi = pos0 + t;
            if (j0 > pi || j0 + TK - 1 < pi - d.window + 1) continue;
            float s = 0.f;
            for (int g = 0; g < H; ++g) s = fmaf(Ts[h * H + g], Ss[(t * H + g) * 32 + lane], s);
            const int j = j0 + lane;
            const bool ok = lane < TK && j <= pi && pi - j < d.window;
            const float tile_max = warp_max(ok ? s : -INFINITY);
            const float m_new = fmaxf(mx[t], tile_max);
            const float p = ok ? expf(s - m_new) : 0.f;
            const float corr = mx[t] == -INFINITY ? 0.f : expf(mx[t] - m_new);
            sum[t] = sum[t] * corr + warp_sum(p);
            mx[t] = m_new;
#pragma unroll
            for (int i = 0; i < DVL; ++i) O[t][i] *= corr;
            const float* vb = Vs + kvh * dv + lane;
            for (int k = 0; k < TK; ++k) {
                const float pk = __shfl_sync(0xffffffffu, p, k);
                if (pk == 0.f) continue;       // uniform over the warp
#pragma unroll
                for (int i = 0; i < DVL; ++i)
                    if (lane + 32 * i < dv) O[t][i] = fmaf(pk, vb[k * G * dv + 32 * i], O[t][i]);
            }
        }
    }
#pragma unroll
    for (int t = 0; t < TA_TQ; ++t) {
        if (t >= nq) break;
        const float r = out_scale / sum[t];
#pragma unroll
        for (int i = 0; i < DVL; ++i)
            if (lane + 32 * i < dv) stx(out, (long long)(t0 + t) * ldo + (long long)h * dv + lane + 32 * i, of32, O[t][i] * r);
    }
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
                          const PagedRows& cache, void* out, int of32, long long ldo, float out_scale, cudaStream_t stream) {
    if (ix.M <= 0 || nseq <= 0) return 0;
    (void)max_kv_len;
    if (d.heads <= 0 || d.heads > 32 || d.kv_heads <= 0 || d.heads % d.kv_heads)
        return set_error("talk_attention: %d heads (at most 32) over %d key/value heads", d.heads, d.kv_heads);
    if (d.dv > 256 || d.dv <= 0 || d.dk <= 0 || d.window <= 0) return set_error("talk_attention: bad sizes");
    // the largest tile that fits shared memory; it depends on the layer's sizes alone, never on the batch
    static const int kTiles[][2] = {{8, 32}, {4, 32}, {8, 16}, {2, 32}, {4, 16}, {1, 32}, {2, 16}, {1, 16}, {1, 8}, {1, 4}, {1, 2}, {1, 1}};
    TalkTile tl{0, 0, 0};
    size_t smem = 0;
    const int tq_max = d.heads > 16 ? 2 : 8;
    for (const auto& c : kTiles) {
        if (c[0] > tq_max) continue;
        const int ks = (d.kv_heads * d.dk) | 1;
        const size_t need = ((size_t)c[0] * d.heads * d.dk + (size_t)c[1] * ks + (size_t)c[1] * d.kv_heads * d.dv +
                             (size_t)c[0] * d.heads * 32 + (size_t)d.heads * d.heads) * sizeof(float);
        if (need <= 200 * 1024) {
            tl = TalkTile{c[0], c[1], ks};
            smem = need;
            break;
        }
    }
    if (!tl.tq) return set_error("talk_attention: the heads' rows do not fit shared memory");
    dim3 grid((max_qlen + tl.tq - 1) / tl.tq, nseq);
    if (grid.y > 65535) return set_error("talk_attention: too many sequences");
    const int dvl = (d.dv + 31) / 32;
#define ASD_TA_CASE2(L, Q)                                                                                            \
    {                                                                                                                 \
        auto fn = talk_attention_kernel<L, Q>;                                                                        \
        static PerDeviceOnce once;                                                                                    \
        if (once.need()) ASD_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024)); \
        fn<<<grid, d.heads * 32, smem, stream>>>(ix, cu_q, seq_slot, q, ldq, d, talk, sink, cache, out, of32, ldo,     \
                                                 out_scale, tl);                                                      \
    }
#define ASD_TA_CASE(L)                     \
    if (tq_max == 8) ASD_TA_CASE2(L, 8)    \
    else ASD_TA_CASE2(L, 2)
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
    count_launch(1);
    ASD_CUDA(cudaGetLastError());
    return 0;
}

}  // namespace asd
