// Delta-rule recurrences: per head a state S [dk][dv] in fp32 that every position decays per key channel, corrects along
// one direction and writes into,
//   gated delta rule:        S' = diag(g) S;  u = beta (v - S'^T k);  S = S' + k u^T;          o = S^T q
//   generalised delta rule:  S  = diag(w) S_old - (a * n)(n^T S_old) + k v^T, n the unit key;  o = S^T r
// and the row kernels around them: channel functions of a low-rank projection (decays, gates), the short causal
// convolution with its carried inputs, the preparation of a position's vectors, the per-head norm and gate of the result.
//
// Both rules are one kernel with one exchange per position.  Generalised rule: a step reads the state it starts from
// through two dot products per value column, A = sum_r S[r] n[r] and B = sum_r S[r] (w * r)[r], and then updates
// S[r] <- w[r] S[r] - (a * n)[r] A + k[r] v, while o = B - A s1 + v s2 with s1 = (a * n) . r, s2 = k . r (the read-out
// of the updated state is expanded, so that one pass over the old state serves the correction and the result); five
// vectors per position (w, n, w * r, k, a * n).  Gated rule, in the order it is written: S[r] <- g[r] S[r], then
// A = sum_r S[r] k[r] and B = sum_r S[r] q[r] in the same pass, u = beta (v - A), S[r] <- S[r] + k[r] u (k still in
// registers: nothing is read after the exchange), o = B + u (k . q); three vectors per position (g, k, q).  delta_prep_kernel forms these vectors; delta_recurrence_kernel holds a CTA's 32 value columns of the state
// in registers, the key rows cut into slices over its warps, for the whole run of new positions.  The arithmetic per
// position is the same whatever the chunking or the batch.  State: fp32 [slot][ring][head][dk][dv], entry p % ring =
// the state after position p.
#include <cuda_bf16.h>

#include "asd_internal.h"
#include "blocks.h"
#include "elem.cuh"

namespace asd {

namespace {

// ------------------------------------------------------------------------------------------ low-rank channel functions
constexpr int LC_TOK = 32, LC_CH = 256;   // tokens x channels per CTA

__device__ __forceinline__ float softplus_f(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }
__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }

// One CTA = 256 channels x 32 tokens: the channels' rows of the second matrix are staged transposed ([low][256]) and
// reused for all the tile's tokens, whose inner vectors every thread reads as broadcasts.
__global__ void __launch_bounds__(LC_CH) lowrank_channels_kernel(const float* a, long long lda, LowRankChannels p, float* out,
                                                                 int M) {
    extern __shared__ float sm[];
    float* wT = sm;                      // [low][LC_CH]
    float* av = sm + p.low * LC_CH;      // [LC_TOK][low]
    const int n = p.n;
    const int c0 = blockIdx.x * LC_CH, m0 = blockIdx.y * LC_TOK;
    const int nt = min(LC_TOK, M - m0);
    // unrolled: eight independent loads in flight per thread instead of a load-then-store chain
#pragma unroll 8
    for (int i = threadIdx.x; i < LC_CH * p.low; i += LC_CH) {
        const int c = i / p.low, r = i - c * p.low;
        wT[r * LC_CH + c] = c0 + c < n ? __ldg(p.w2 + (long long)(c0 + c) * p.low + r) : 0.f;
    }
#pragma unroll 4
    for (int i = threadIdx.x; i < LC_TOK * p.low; i += LC_CH) {
        const int t = i / p.low, r = i - t * p.low;
        float v = t < nt ? __ldg(a + (long long)(m0 + t) * lda + r) : 0.f;
        if (p.inner_tanh) v = tanhf(v);
        av[i] = v;
    }
    __syncthreads();
    const int c = c0 + threadIdx.x;
    if (c >= n) return;
    float z[LC_TOK];
#pragma unroll
    for (int t = 0; t < LC_TOK; ++t) z[t] = 0.f;
    for (int r = 0; r < p.low; ++r) {
        const float w = wT[r * LC_CH + threadIdx.x];
#pragma unroll
        for (int t = 0; t < LC_TOK; ++t) z[t] = fmaf(w, av[t * p.low + r], z[t]);
    }
    const float bias = p.bias ? p.bias[c] : 0.f;
    const float rate = p.post == LRC_EXP_SOFTPLUS ? expf(p.head_log_rate[c / p.per_head]) : p.rate;
#pragma unroll
    for (int t = 0; t < LC_TOK; ++t) {
        if (t < nt) {
            const float zz = z[t] + bias;
            float v;
            // a slow decay lies just below 1, where expf's error is a relative 1e-7 that hundreds of steps multiply;
            // 1 + expm1 is rounded once
            if (p.post == LRC_EXP_SOFTPLUS)
                v = 1.f + expm1f(-rate * softplus_f(zz));
            else if (p.post == LRC_EXP_SIGMOID)
                v = 1.f + expm1f(-rate * sigmoid_f(zz));
            else
                v = sigmoid_f(zz);
            out[(long long)(m0 + t) * n + c] = v;
        }
    }
}

// ------------------------------------------------------------------------------------------ short causal convolution
// out[m][c] = silu( sum_j taps[c][j] * in[position - (n - 1 - j)][c] ): inputs of this forward come from the rows above
// (a sequence's tokens are consecutive rows), earlier ones from the ring of carried inputs, zeros before position 0.
__global__ void short_conv_kernel(SeqIndex ix, const float* in, long long ld, const float* taps, int n, int C,
                                  const float* ring, int ring_n, float* out) {
    const int m = blockIdx.x;
    const int pos = ix.positions[m], slot = ix.token_slot[m];
    // how many rows above belong to the same sequence's preceding positions (at most n - 1 are needed)
    int above = 0;
    while (above < n - 1 && m - above - 1 >= 0 && ix.token_slot[m - above - 1] == slot &&
           ix.positions[m - above - 1] == pos - above - 1)
        ++above;
    // four channels per thread, blockDim apart, their loads independent of one another
    const int cb = blockIdx.y * blockDim.x * 4 + threadIdx.x;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < n; ++j) {
        const int back = n - 1 - j;       // taps' last column weighs the current position
        const int p = pos - back;
        if (p < 0) continue;
        const float* src = back <= above ? in + (long long)(m - back) * ld : ring + ((long long)slot * ring_n + p % ring_n) * C;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int c = cb + u * blockDim.x;
            if (c < C) acc[u] = fmaf(__ldg(taps + (long long)c * n + j), __ldg(src + c), acc[u]);
        }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const int c = cb + u * blockDim.x;
        if (c < C) out[(long long)m * C + c] = acc[u] / (1.f + expf(-acc[u]));
    }
}

// the last ring_n new positions of every sequence leave their inputs behind (runs after short_conv_kernel has read)
__global__ void conv_commit_kernel(SeqIndex ix, const int* cu_q, const float* in, long long ld, int C, float* ring,
                                   int ring_n) {
    const int seq = blockIdx.x;
    const int t1 = cu_q[seq + 1], t0 = max(cu_q[seq], t1 - ring_n);
    for (int m = t0 + blockIdx.y; m < t1; m += gridDim.y) {
        const int pos = ix.positions[m], slot = ix.token_slot[m];
        float* dst = ring + ((long long)slot * ring_n + pos % ring_n) * C;
#pragma unroll 8
        for (int c = threadIdx.x; c < C; c += blockDim.x) dst[c] = __ldg(in + (long long)m * ld + c);
    }
}

// ------------------------------------------------------------------------------------------ a position's vectors
// one warp per (token, head): rv[m][h][vec][dk] with vec = g, k, q (gated) or w, n, w * r, k, a * n (generalised) and
// sc[m][h][4] = beta, -, k . q, - (gated) or -, -, (a * n) . r, k . r (generalised)
__global__ void delta_prep_kernel(DeltaPrep p, int M) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long idx = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
    if (idx >= (long long)M * p.heads) return;
    const int m = (int)(idx / p.heads), h = (int)(idx - (long long)m * p.heads);
    const int dk = p.dk, nv = p.general ? 5 : 3;
    const int kvh = h / (p.heads / p.kv_heads);
    const float* q = p.q + (long long)m * p.ld + (long long)kvh * dk;
    const float* k = p.k + (long long)m * p.ld + (long long)kvh * dk;
    const float* d = p.decay + ((long long)m * p.heads + h) * dk;
    float* rv = p.rv + ((long long)m * p.heads + h) * nv * dk;
    float kk = 0.f, qq = 0.f;
    for (int i = lane; i < dk; i += 32) {
        kk = fmaf(k[i], k[i], kk);
        qq = fmaf(q[i], q[i], qq);
    }
    kk = warp_sum(kk);
    qq = warp_sum(qq);
    const float kn = 1.f / sqrtf(kk + p.tiny);
    float s1 = 0.f, s2 = 0.f;
    if (!p.general) {
        const float qn = p.q_scale / sqrtf(qq + p.tiny);
        for (int i = lane; i < dk; i += 32) {
            const float kv = k[i] * kn, qv = q[i] * qn, dv = d[i];
            rv[i] = dv;
            rv[dk + i] = kv;
            rv[2 * dk + i] = qv;
            s1 = fmaf(kv, qv, s1);
        }
        s1 = warp_sum(s1);
        if (lane == 0) {
            const float beta = sigmoid_f(p.beta[(long long)m * p.ld_beta + h]);
            float* sc = p.sc + ((long long)m * p.heads + h) * 4;
            sc[0] = beta, sc[1] = beta, sc[2] = s1, sc[3] = s1;
        }
    } else {
        const float* a = p.rate + (long long)m * p.ld + (long long)h * dk;
        const float* ab = p.rate_bias + (long long)h * dk;
        for (int i = lane; i < dk; i += 32) {
            const float kv = k[i], nvv = kv * kn, rr = q[i], dv = d[i];
            const float an = sigmoid_f(a[i] + ab[i]) * nvv;
            rv[i] = dv;
            rv[dk + i] = nvv;
            rv[2 * dk + i] = dv * rr;
            rv[3 * dk + i] = kv;
            rv[4 * dk + i] = an;
            s1 = fmaf(an, rr, s1);
            s2 = fmaf(kv, rr, s2);
        }
        s1 = warp_sum(s1);
        s2 = warp_sum(s2);
        if (lane == 0) {
            float* sc = p.sc + ((long long)m * p.heads + h) * 4;
            sc[0] = 1.f, sc[1] = 1.f, sc[2] = s1, sc[3] = s2;
        }
    }
}

// ------------------------------------------------------------------------------------------ the recurrence
__device__ __forceinline__ void cp_async4z(float* dst, const float* src, bool valid) {
    const unsigned addr = (unsigned)__cvta_generic_to_shared(dst);
    const int sz = valid ? 4 : 0;       // 0: the destination is filled with zeros
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(addr), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async16(float* dst, const float* src) {
    const unsigned addr = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(addr), "l"(src) : "memory");
}

// ROWS state rows per thread; warps = slices of ROWS key rows (rows beyond dk are staged as zeros and keep a zero
// state).  NV = 3: the gated rule; NV = 5: the generalised rule.  CH positions are staged per chunk by
// cp.async, one chunk ahead of the arithmetic.
template <int ROWS, int NV, int MAXT>
__global__ void __launch_bounds__(MAXT, 1) delta_recurrence_kernel(SeqIndex ix, const int* cu_q, const int* seq_slot,
                                                                   const float* rv, const float* sc, const float* v,
                                                                   long long ldv, int heads, int dk, int dv, float* state,
                                                                   int ring, float* out, int CH) {
    extern __shared__ __align__(16) float sm[];
    const int seq = blockIdx.x, head = blockIdx.y, col0 = blockIdx.z * 32;
    const int t0 = cu_q[seq], t1 = cu_q[seq + 1];
    if (t0 >= t1) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, RS = blockDim.x >> 5, nthr = blockDim.x;
    const int dkp = RS * ROWS, r0 = warp * ROWS;
    const int col = col0 + lane;
    const bool col_ok = col < dv;
    const int slot = seq_slot[seq];
    const int p0 = ix.positions[t0];
    // shared: two buffers of { vectors [CH][NV][dkp], v [CH][32], scalars [CH][4] }, then the partial sums [2][RS][2][32]
    const int buf_elems = CH * NV * dkp + CH * 36;
    float* red = sm + 2 * buf_elems;
    for (int i = threadIdx.x; i < 2 * buf_elems; i += nthr) sm[i] = 0.f;   // key rows beyond dk stay zero for good
    const long long st_head = ((long long)head * dk) * dv;
    const long long st_entry = (long long)heads * dk * dv;
    float* st_slot = state + (long long)slot * ring * st_entry;
    float S[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) S[r] = 0.f;
    if (p0 > 0 && col_ok) {
        const float* src = st_slot + (long long)((p0 - 1) % ring) * st_entry + st_head;
#pragma unroll
        for (int r = 0; r < ROWS; ++r)
            if (r0 + r < dk) S[r] = src[(long long)(r0 + r) * dv + col];
    }
    const int hv = head * dv;
    const bool v16 = (dk & 3) == 0;     // a (token, head)'s vectors then start on 16-byte boundaries
    __syncthreads();
    auto fetch = [&](int buf, int c0) {
        const int nt = min(CH, t1 - c0);
        float* vec = sm + buf * buf_elems;
        float* vs = vec + CH * NV * dkp;
        float* ss = vs + CH * 32;
        if (v16) {
            const int n4 = dk >> 2, per = NV * n4;
            for (int i = threadIdx.x; i < nt * per; i += nthr) {
                const int t = i / per, rest = i - t * per;
                const int j = rest / n4, c4 = rest - j * n4;
                cp_async16(vec + (t * NV + j) * dkp + 4 * c4, rv + (((long long)(c0 + t) * heads + head) * NV + j) * dk + 4 * c4);
            }
        } else {
            const int per = NV * dk;
            for (int i = threadIdx.x; i < nt * per; i += nthr) {
                const int t = i / per, rest = i - t * per;
                const int j = rest / dk, c = rest - j * dk;
                cp_async4z(vec + (t * NV + j) * dkp + c, rv + (((long long)(c0 + t) * heads + head) * NV + j) * dk + c, true);
            }
        }
        for (int i = threadIdx.x; i < nt * 32; i += nthr) {
            const int t = i >> 5, c = i & 31;
            const bool ok = col0 + c < dv;
            cp_async4z(vs + i, v + (ok ? (long long)(c0 + t) * ldv + hv + col0 + c : 0), ok);
        }
        for (int i = threadIdx.x; i < nt * 4; i += nthr)
            cp_async4z(ss + i, sc + ((long long)(c0 + (i >> 2)) * heads + head) * 4 + (i & 3), true);
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    fetch(0, t0);
    int par = 0, it = 0;
    for (int c0 = t0; c0 < t1; c0 += CH, ++it) {
        const int nt = min(CH, t1 - c0);
        if (c0 + CH < t1) {
            fetch((it + 1) & 1, c0 + CH);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();   // this chunk's rows have landed for every thread
        const float* vec = sm + (it & 1) * buf_elems;
        const float* vs = vec + CH * NV * dkp;
        const float* ss = vs + CH * 32;
        for (int t = 0; t < nt; ++t, par ^= 1) {
            const float* vt = vec + t * NV * dkp + r0;
            const float4* d4 = reinterpret_cast<const float4*>(vt);
            float* rp = red + (size_t)par * RS * 64;
            float o_t;
            if constexpr (NV == 3) {
                const float4* k4 = reinterpret_cast<const float4*>(vt + dkp);
                const float4* q4 = reinterpret_cast<const float4*>(vt + 2 * dkp);
                float kr[ROWS];
                float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
#pragma unroll
                for (int r = 0; r < ROWS; r += 4) {
                    const float4 dd = d4[r >> 2], kk = k4[r >> 2], qq = q4[r >> 2];
                    kr[r] = kk.x, kr[r + 1] = kk.y, kr[r + 2] = kk.z, kr[r + 3] = kk.w;
                    S[r] *= dd.x, S[r + 1] *= dd.y, S[r + 2] *= dd.z, S[r + 3] *= dd.w;
                    a0 = fmaf(S[r], kk.x, a0);
                    a1 = fmaf(S[r + 1], kk.y, a1);
                    a0 = fmaf(S[r + 2], kk.z, a0);
                    a1 = fmaf(S[r + 3], kk.w, a1);
                    b0 = fmaf(S[r], qq.x, b0);
                    b1 = fmaf(S[r + 1], qq.y, b1);
                    b0 = fmaf(S[r + 2], qq.z, b0);
                    b1 = fmaf(S[r + 3], qq.w, b1);
                }
                rp[warp * 64 + lane] = a0 + a1;
                rp[warp * 64 + 32 + lane] = b0 + b1;
                __syncthreads();
                float A = 0.f, B = 0.f;
                for (int w = 0; w < RS; ++w) {      // every warp adds the slices in index order: the same totals everywhere
                    A += rp[w * 64 + lane];
                    B += rp[w * 64 + 32 + lane];
                }
                const float u = ss[t * 4 + 0] * (vs[t * 32 + lane] - A);
#pragma unroll
                for (int r = 0; r < ROWS; ++r) S[r] = fmaf(kr[r], u, S[r]);
                o_t = fmaf(u, ss[t * 4 + 2], B);
            } else {
            const float4* x14 = reinterpret_cast<const float4*>(vt + dkp);
            const float4* x24 = reinterpret_cast<const float4*>(vt + 2 * dkp);
            const float4* k4 = reinterpret_cast<const float4*>(vt + 3 * dkp);
            const float4* y4 = reinterpret_cast<const float4*>(vt + 4 * dkp);
            float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
#pragma unroll
            for (int r = 0; r < ROWS; r += 4) {
                const float4 x = x14[r >> 2], z = x24[r >> 2];
                a0 = fmaf(S[r], x.x, a0);
                a1 = fmaf(S[r + 1], x.y, a1);
                a0 = fmaf(S[r + 2], x.z, a0);
                a1 = fmaf(S[r + 3], x.w, a1);
                b0 = fmaf(S[r], z.x, b0);
                b1 = fmaf(S[r + 1], z.y, b1);
                b0 = fmaf(S[r + 2], z.z, b0);
                b1 = fmaf(S[r + 3], z.w, b1);
            }
            rp[warp * 64 + lane] = a0 + a1;
            rp[warp * 64 + 32 + lane] = b0 + b1;
            __syncthreads();
            float A = 0.f, B = 0.f;
            for (int w = 0; w < RS; ++w) {      // every warp adds the slices in index order: the same totals everywhere
                A += rp[w * 64 + lane];
                B += rp[w * 64 + 32 + lane];
            }
            const float vv = vs[t * 32 + lane];
            const float cA = -A, cB = vv;
#pragma unroll
            for (int r = 0; r < ROWS; r += 4) {
                const float4 dd = d4[r >> 2], kk = k4[r >> 2], yy = y4[r >> 2];
                S[r] = fmaf(kk.x, cB, fmaf(yy.x, cA, dd.x * S[r]));
                S[r + 1] = fmaf(kk.y, cB, fmaf(yy.y, cA, dd.y * S[r + 1]));
                S[r + 2] = fmaf(kk.z, cB, fmaf(yy.z, cA, dd.z * S[r + 2]));
                S[r + 3] = fmaf(kk.w, cB, fmaf(yy.w, cA, dd.w * S[r + 3]));
            }
            o_t = fmaf(cB, ss[t * 4 + 3], fmaf(cA, ss[t * 4 + 2], B));
            }
            const int m = c0 + t;
            if (warp == 0 && col_ok) out[(long long)m * heads * dv + hv + col] = o_t;
            if (t1 - m <= ring && col_ok) {     // the last `ring` new positions leave their state behind
                float* dst = st_slot + (long long)((p0 + (m - t0)) % ring) * st_entry + st_head;
#pragma unroll
                for (int r = 0; r < ROWS; ++r)
                    if (r0 + r < dk) dst[(long long)(r0 + r) * dv + col] = S[r];
            }
        }
        __syncthreads();   // the chunk is consumed: its buffer may be refilled
    }
}

// Key sizes up to 128: PARTS neighbouring lanes share a value column, each holding 32 key rows of it in registers, so
// that the two dot products are closed by shuffles among those lanes and a position costs no barrier: the warps of a
// CTA (one per 32 / PARTS columns of one (sequence, head)) only meet when a chunk of staged positions is used up.
template <int PARTS, int NV>
__global__ void __launch_bounds__(512, 1) delta_recurrence_cols_kernel(SeqIndex ix, const int* cu_q, const int* seq_slot,
                                                                       const float* rv, const float* sc, const float* v,
                                                                       long long ldv, int heads, int dk, int dv, float* state,
                                                                       int ring, float* out, int CH) {
    constexpr int ROWS = 32, PS = 36, DKP = PS * PARTS;   // a row block's staged floats start PS apart: the blocks'
                                                           // 16-byte reads fall into different banks
    extern __shared__ __align__(16) float sm[];
    const int seq = blockIdx.x, head = blockIdx.y;
    const int t0 = cu_q[seq], t1 = cu_q[seq + 1];
    if (t0 >= t1) return;
    const int nthr = blockDim.x, dvp = nthr / PARTS;     // value columns padded to whole warps
    const int col = threadIdx.x / PARTS, part = threadIdx.x % PARTS, r0 = part * ROWS;
    const bool col_ok = col < dv;
    const int slot = seq_slot[seq];
    const int p0 = ix.positions[t0];
    // shared: two buffers of { vectors [CH][NV][DKP], v [CH][dvp], scalars [CH][4] }
    const int buf_elems = CH * NV * DKP + CH * dvp + CH * 4;
    for (int i = threadIdx.x; i < 2 * buf_elems; i += nthr) sm[i] = 0.f;   // key rows beyond dk stay zero for good
    const long long st_head = ((long long)head * dk) * dv;
    const long long st_entry = (long long)heads * dk * dv;
    float* st_slot = state + (long long)slot * ring * st_entry;
    float S[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) S[r] = 0.f;
    if (p0 > 0 && col_ok) {
        const float* src = st_slot + (long long)((p0 - 1) % ring) * st_entry + st_head;
#pragma unroll
        for (int r = 0; r < ROWS; ++r)
            if (r0 + r < dk) S[r] = src[(long long)(r0 + r) * dv + col];
    }
    const int hv = head * dv;
    const bool v16 = (dk & 3) == 0;
    __syncthreads();
    auto fetch = [&](int buf, int c0) {
        const int nt = min(CH, t1 - c0);
        float* vec = sm + buf * buf_elems;
        float* vs = vec + CH * NV * DKP;
        float* ss = vs + CH * dvp;
        if (v16) {
            const int n4 = dk >> 2, per = NV * n4;
            for (int i = threadIdx.x; i < nt * per; i += nthr) {
                const int t = i / per, rest = i - t * per;
                const int j = rest / n4, c4 = rest - j * n4;
                cp_async16(vec + (t * NV + j) * DKP + (c4 >> 3) * PS + 4 * (c4 & 7), rv + (((long long)(c0 + t) * heads + head) * NV + j) * dk + 4 * c4);
            }
        } else {
            const int per = NV * dk;
            for (int i = threadIdx.x; i < nt * per; i += nthr) {
                const int t = i / per, rest = i - t * per;
                const int j = rest / dk, c = rest - j * dk;
                cp_async4z(vec + (t * NV + j) * DKP + (c >> 5) * PS + (c & 31), rv + (((long long)(c0 + t) * heads + head) * NV + j) * dk + c, true);
            }
        }
        for (int i = threadIdx.x; i < nt * dvp; i += nthr) {
            const int t = i / dvp, c = i - t * dvp;
            const bool ok = c < dv;
            cp_async4z(vs + i, v + (ok ? (long long)(c0 + t) * ldv + hv + c : 0), ok);
        }
        for (int i = threadIdx.x; i < nt * 4; i += nthr)
            cp_async4z(ss + i, sc + ((long long)(c0 + (i >> 2)) * heads + head) * 4 + (i & 3), true);
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    fetch(0, t0);
    int it = 0;
    for (int c0 = t0; c0 < t1; c0 += CH, ++it) {
        const int nt = min(CH, t1 - c0);
        if (c0 + CH < t1) {
            fetch((it + 1) & 1, c0 + CH);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();   // this chunk's rows have landed for every thread
        const float* vec = sm + (it & 1) * buf_elems;
        const float* vs = vec + CH * NV * DKP;
        const float* ss = vs + CH * dvp;
        for (int t = 0; t < nt; ++t) {
            const float4* d4 = reinterpret_cast<const float4*>(vec + t * NV * DKP + part * PS);
            float o_t;
            if constexpr (NV == 3) {
                const float4* k4 = d4 + DKP / 4;
                const float4* q4 = d4 + 2 * (DKP / 4);
                float kr[ROWS];
                float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
#pragma unroll
                for (int r = 0; r < ROWS; r += 4) {
                    const float4 dd = d4[r >> 2], kk = k4[r >> 2], qq = q4[r >> 2];
                    kr[r] = kk.x, kr[r + 1] = kk.y, kr[r + 2] = kk.z, kr[r + 3] = kk.w;
                    S[r] *= dd.x, S[r + 1] *= dd.y, S[r + 2] *= dd.z, S[r + 3] *= dd.w;
                    a0 = fmaf(S[r], kk.x, a0);
                    a1 = fmaf(S[r + 1], kk.y, a1);
                    a0 = fmaf(S[r + 2], kk.z, a0);
                    a1 = fmaf(S[r + 3], kk.w, a1);
                    b0 = fmaf(S[r], qq.x, b0);
                    b1 = fmaf(S[r + 1], qq.y, b1);
                    b0 = fmaf(S[r + 2], qq.z, b0);
                    b1 = fmaf(S[r + 3], qq.w, b1);
                }
                float A = a0 + a1, B = b0 + b1;
#pragma unroll
                for (int o = 1; o < PARTS; o <<= 1) {
                    A += __shfl_xor_sync(0xffffffffu, A, o);
                    B += __shfl_xor_sync(0xffffffffu, B, o);
                }
                const float u = ss[t * 4 + 0] * (vs[t * dvp + col] - A);
#pragma unroll
                for (int r = 0; r < ROWS; ++r) S[r] = fmaf(kr[r], u, S[r]);
                o_t = fmaf(u, ss[t * 4 + 2], B);
            } else {
            const float4* x14 = d4 + DKP / 4;
            const float4* x24 = d4 + 2 * (DKP / 4);
            const float4* k4 = d4 + 3 * (DKP / 4);
            const float4* y4 = d4 + 4 * (DKP / 4);
            float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f, b0 = 0.f, b1 = 0.f, b2 = 0.f, b3 = 0.f;
#pragma unroll
            for (int r = 0; r < ROWS; r += 4) {
                const float4 x = x14[r >> 2], z = x24[r >> 2];
                a0 = fmaf(S[r], x.x, a0);
                a1 = fmaf(S[r + 1], x.y, a1);
                a2 = fmaf(S[r + 2], x.z, a2);
                a3 = fmaf(S[r + 3], x.w, a3);
                b0 = fmaf(S[r], z.x, b0);
                b1 = fmaf(S[r + 1], z.y, b1);
                b2 = fmaf(S[r + 2], z.z, b2);
                b3 = fmaf(S[r + 3], z.w, b3);
            }
            float A = (a0 + a1) + (a2 + a3), B = (b0 + b1) + (b2 + b3);
#pragma unroll
            for (int o = 1; o < PARTS; o <<= 1) {       // the column's other row blocks: the same total in every lane
                A += __shfl_xor_sync(0xffffffffu, A, o);
                B += __shfl_xor_sync(0xffffffffu, B, o);
            }
            const float vv = vs[t * dvp + col];
            const float cA = -A, cB = vv;
#pragma unroll
            for (int r = 0; r < ROWS; r += 4) {
                const float4 dd = d4[r >> 2], kk = k4[r >> 2], yy = y4[r >> 2];
                S[r] = fmaf(kk.x, cB, fmaf(yy.x, cA, dd.x * S[r]));
                S[r + 1] = fmaf(kk.y, cB, fmaf(yy.y, cA, dd.y * S[r + 1]));
                S[r + 2] = fmaf(kk.z, cB, fmaf(yy.z, cA, dd.z * S[r + 2]));
                S[r + 3] = fmaf(kk.w, cB, fmaf(yy.w, cA, dd.w * S[r + 3]));
            }
            o_t = fmaf(cB, ss[t * 4 + 3], fmaf(cA, ss[t * 4 + 2], B));
            }
            const int m = c0 + t;
            if (col_ok && part == 0) out[(long long)m * heads * dv + hv + col] = o_t;
            if (t1 - m <= ring && col_ok) {     // the last `ring` new positions leave their state behind
                float* dst = st_slot + (long long)((p0 + (m - t0)) % ring) * st_entry + st_head;
#pragma unroll
                for (int r = 0; r < ROWS; ++r)
                    if (r0 + r < dk) dst[(long long)(r0 + r) * dv + col] = S[r];
            }
        }
        __syncthreads();   // the chunk is consumed: its buffer may be refilled
    }
}

// ------------------------------------------------------------------------------------------ norm and gate of the result
// one warp per (token, head): y = o / rms(o over dv) * w * gate * scale
__global__ void head_norm_gate_kernel(const float* o, HeadNormGate p, void* y, int of32, long long ldy, int heads, int dv) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.y * (blockDim.x >> 5) + warp;
    if (h >= heads) return;
    const long long m = blockIdx.x;
    const float* src = o + (m * heads + h) * dv;
    const float* g = p.gate + m * p.ldg + (long long)h * dv;
    const float* w = p.w + (p.w_per_head ? (long long)h * dv : 0);
    float ss = 0.f;
    for (int i = lane; i < dv; i += 32) ss = fmaf(src[i], src[i], ss);
    ss = warp_sum(ss);
    const float r = p.scale / sqrtf(ss / (float)dv + p.eps);
    for (int i = lane; i < dv; i += 32) {
        const float gv = p.gate_sigmoid ? sigmoid_f(g[i]) : g[i];
        stx(y, m * ldy + (long long)h * dv + i, of32, src[i] * r * w[i] * gv);
    }
}

}  // namespace

int launch_lowrank_channels(const float* a, long long lda, const LowRankChannels& p, float* out, int M, cudaStream_t stream) {
    if (M <= 0 || p.n <= 0) return 0;
    if (p.low <= 0 || !p.w2) return set_error("lowrank_channels: no inner projection");
    if (p.post == LRC_EXP_SOFTPLUS && (!p.head_log_rate || p.per_head <= 0))
        return set_error("lowrank_channels: the per-head rates are missing");
    const size_t smem = (size_t)p.low * (LC_CH + LC_TOK) * sizeof(float);
    if (smem > 200 * 1024) return set_error("lowrank_channels: inner size %d does not fit shared memory", p.low);
    static PerDeviceOnce once;
    if (once.need())
        ASD_CUDA(cudaFuncSetAttribute(lowrank_channels_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
    dim3 grid((p.n + LC_CH - 1) / LC_CH, (M + LC_TOK - 1) / LC_TOK);
    if (grid.y > 65535) return set_error("lowrank_channels: too many tokens");
    lowrank_channels_kernel<<<grid, LC_CH, smem, stream>>>(a, lda, p, out, M);
    count_launch(1);
    ASD_CUDA(cudaGetLastError());
    return 0;
}

int launch_short_conv(const SeqIndex& ix, const float* in, long long ld, const float* taps, int n_taps, int C,
                      const float* ring, int ring_n, float* out, cudaStream_t stream) {
    if (ix.M <= 0 || C <= 0) return 0;
    if (n_taps <= 0 || (n_taps > 1 && (!ring || ring_n < n_taps - 1)))
        return set_error("short_conv: %d taps need a ring of at least %d carried inputs", n_taps, n_taps - 1);
    const int threads = C >= 1024 ? 256 : 128;
    dim3 grid(ix.M, (C + 4 * threads - 1) / (4 * threads));
    if (grid.y > 65535) return set_error("short_conv: too many channels");
    short_conv_kernel<<<grid, threads, 0, stream>>>(ix, in, ld, taps, n_taps, C, ring, ring_n > 0 ? ring_n : 1, out);
    count_launch(1);
    ASD_CUDA(cudaGetLastError());
    return 0;
}

int launch_conv_commit(const SeqIndex& ix, const int* cu_q, int nseq, const float* in, long long ld, int C, float* ring,
                       int ring_n, cudaStream_t stream) {
    if (ix.M <= 0 || nseq <= 0 || ring_n <= 0 || C <= 0) return 0;
    dim3 grid(nseq, ring_n < 16 ? ring_n : 16);
    conv_commit_kernel<<<grid, C >= 1024 ? 256 : 128, 0, stream>>>(ix, cu_q, in, ld, C, ring, ring_n);
    count_launch(1);
    ASD_CUDA(cudaGetLastError());
    return 0;
}

int launch_delta_prep(const DeltaPrep& p, int M, cudaStream_t stream) {
    if (M <= 0) return 0;
    if (p.heads <= 0 || p.kv_heads <= 0 || p.heads % p.kv_heads || p.dk <= 0)
        return set_error("delta_prep: %d heads over %d key heads of size %d", p.heads, p.kv_heads, p.dk);
    if (p.general ? (!p.rate || !p.rate_bias) : !p.beta) return set_error("delta_prep: missing inputs");
    const long long pairs = (long long)M * p.heads;
    delta_prep_kernel<<<(unsigned)((pairs + 7) / 8), 256, 0, stream>>>(p, M);
    count_launch(1);
    ASD_CUDA(cudaGetLastError());
    return 0;
}

int launch_delta_recurrence(const SeqIndex& ix, const int* cu_q, const int* seq_slot, int nseq, const float* rv,
                            const float* sc, int general, const float* v, long long ldv, int heads, int dk, int dv,
                            float* state, int ring, float* out, cudaStream_t stream) {
    if (ix.M <= 0 || nseq <= 0) return 0;
    if (dk <= 0 || dk > 1024) return set_error("delta rule: key size %d outside 1..1024", dk);
    if (ring <= 0 || !state) return set_error("delta rule: no state");
    const int parts = dk <= 32 ? 1 : (dk <= 64 ? 2 : 4);
    // steps of single tokens: the state is read and written once per position and the shuffle form keeps more loads in
    // flight; prompts and portions: the slices over warps read every staged vector once per warp as a broadcast
    if (ix.M <= 2 * nseq && dk <= 128 && ((dv + 32 / parts - 1) / (32 / parts)) * 32 <= 512) {   // row blocks closed by shuffles: no barrier per position
        const int nvv = general ? 5 : 3, dkp = 36 * parts;
        const int cpw = 32 / parts, warps = (dv + cpw - 1) / cpw, dvp = warps * cpw;
        int ch = 16;   // positions per staged chunk; steps of few tokens per sequence stage (and clear) no more than they use
        while (ch > 1 && (long long)(ch / 2) * nseq >= ix.M) ch >>= 1;
        auto need = [&](int c) { return (size_t)(2 * (c * nvv * dkp + c * dvp + c * 4)) * sizeof(float); };
        while (ch > 1 && need(ch) > 100 * 1024) ch >>= 1;
        dim3 grid(nseq, heads);
        if (grid.y > 65535) return set_error("delta rule: too many heads");
#define ASD_DC_CASE(P_, NVV)                                                                                           \
    {                                                                                                                 \
        auto fn = delta_recurrence_cols_kernel<P_, NVV>;                                                              \
        static PerDeviceOnce once;                                                                                    \
        if (once.need()) ASD_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024)); \
        fn<<<grid, warps * 32, need(ch), stream>>>(ix, cu_q, seq_slot, rv, sc, v, ldv, heads, dk, dv, state, ring, out, \
                                                   ch);                                                               \
    }
#define ASD_DC_PARTS(NVV)                        \
    if (parts == 1) ASD_DC_CASE(1, NVV)          \
    else if (parts == 2) ASD_DC_CASE(2, NVV)     \
    else ASD_DC_CASE(4, NVV)
        if (general) {
            ASD_DC_PARTS(5)
        } else {
            ASD_DC_PARTS(3)
        }
#undef ASD_DC_PARTS
#undef ASD_DC_CASE
        count_launch(1);
        ASD_CUDA(cudaGetLastError());
        return 0;
    }
    int rows = 4;
    while (rows < 32 && rows * 4 < dk) rows *= 2;     // four warps up to key size 128, then more
    const int RS = (dk + rows - 1) / rows;
    const int dkp = RS * rows, nv = general ? 5 : 3;
    int ch = 16;   // positions per staged chunk: as many as two buffers of a head's vectors leave room for
    while (ch > 1 && (long long)(ch / 2) * nseq >= ix.M) ch >>= 1;
    auto need = [&](int c) { return (size_t)(2 * (c * nv * dkp + c * 36) + 2 * RS * 64) * sizeof(float); };
    while (ch > 1 && need(ch) > 200 * 1024) ch >>= 1;
    const size_t smem = need(ch);
    if (smem > 220 * 1024) return set_error("delta rule: key size %d does not fit shared memory", dk);
    dim3 grid(nseq, heads, (dv + 31) / 32);
    if (grid.y > 65535 || grid.z > 65535) return set_error("delta rule: too many heads or value columns");
#define ASD_DR_CASE(R, NVV, T)                                                                                         \
    {                                                                                                                 \
        auto fn = delta_recurrence_kernel<R, NVV, T>;                                                                  \
        static PerDeviceOnce once;                                                                                    \
        if (once.need()) ASD_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024)); \
        fn<<<grid, RS * 32, smem, stream>>>(ix, cu_q, seq_slot, rv, sc, v, ldv, heads, dk, dv, state, ring, out, ch);  \
    }
#define ASD_DR_ROWS(NVV)                             \
    if (RS > 8) ASD_DR_CASE(32, NVV, 1024)           \
    else if (rows == 4) ASD_DR_CASE(4, NVV, 256)     \
    else if (rows == 8) ASD_DR_CASE(8, NVV, 256)     \
    else if (rows == 16) ASD_DR_CASE(16, NVV, 256)   \
    else ASD_DR_CASE(32, NVV, 256)
    if (general) {
        ASD_DR_ROWS(5)
    } else {
        ASD_DR_ROWS(3)
    }
#undef ASD_DR_ROWS
#undef ASD_DR_CASE
    count_launch(1);
    ASD_CUDA(cudaGetLastError());
    return 0;
}

int launch_head_norm_gate(const float* o, const HeadNormGate& p, void* y, int of32, long long ldy, int M, int heads, int dv,
                          cudaStream_t stream) {
    if (M <= 0) return 0;
    if (!p.w || !p.gate) return set_error("head_norm_gate: missing inputs");
    const int wpb = heads < 8 ? heads : 8;
    dim3 grid(M, (heads + wpb - 1) / wpb);
    head_norm_gate_kernel<<<grid, wpb * 32, 0, stream>>>(o, p, y, of32, ldy, heads, dv);
    count_launch(1);
    ASD_CUDA(cudaGetLastError());
    return 0;
}

}  // namespace asd
