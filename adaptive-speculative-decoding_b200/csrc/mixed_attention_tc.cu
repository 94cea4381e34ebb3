// Mixed-weights attention for prompts and portions of a bf16 engine on the tensor cores (mma.sync m16n8k16, bf16 operands,
// fp32 accumulation).  Same two passes as the CUDA-core kernels (mixed_attention.cu): statistics of every (query, head),
// then normalised weights, their mix across the heads, and the values.  A CTA owns up to 128 (head, query) rows; warp w
// owns rows 16 w .. 16 w + 15, which lie in one key/value group, for the scores, the softmax arithmetic, the mix and the
// values alike.  The fp32 operands (normed queries; softmax weights) enter the tensor cores as two bf16 terms each, so
// that scores and weighted sums keep fp32 accuracy against the cache's bf16 rows; scores, weights and sums are fp32.
// Keys and values of ALL the CTA's key/value groups are staged per key tile (16-byte copies), fragments come through
// ldmatrix.  The mix across the heads goes through shared memory in fp32 and lands directly in A-fragment layout.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include <algorithm>

#include "asd_internal.h"
#include "blocks.h"
#include "elem.cuh"
#include "mixed_attention.h"
#include "mma_sync.cuh"

namespace asd {

namespace {

constexpr int NT = 256;
typedef __nv_bfloat16 bf16;

struct TcLayout {
    int qh, ql, kv, p, talk, m, l, off, total;   // byte offsets, multiples of 16
};
__host__ __device__ inline int up16(int x) { return (x + 15) & ~15; }
__host__ __device__ inline TcLayout tc_layout(int rows, int DS, int VS, int ng, int KT, int heads, bool apply, bool talk,
                                              int nbuf) {
    TcLayout L;
    int o = 0;
    L.qh = o, o += rows * DS * 2;
    L.ql = o, o += rows * DS * 2;
    const int kvw = DS > VS ? DS : VS;
    L.kv = o, o += nbuf * ng * KT * kvw * 2;
    L.p = o, o += (apply && talk) ? rows * (KT + 8) * 4 : 0;
    L.talk = o, o += (apply && talk) ? up16(heads * heads * 4) : 0;
    L.m = o, o += apply ? up16(rows * 4) : 0;
    L.l = o, o += apply ? up16(rows * 4) : 0;
    L.off = o, o += 2 * KT * 8;
    L.total = o;
    return L;
}

// cache rows of the tile's keys, `ng` key/value heads from head_off on (n elements each, hstep apart), -> dst[(group *
// KT + key) * stride + d] for d < np (zeros beyond n and beyond nk)
__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// vec: every 16-byte piece of a row is aligned and whole, so the copies are cp.async (zero-filled beyond the row and
// beyond nk) that the caller commits and waits for; else plain loads and stores, done when the call returns.
template <int KT>
__device__ __forceinline__ void stage_rows(const bf16* pool, const long long* rowoff, int nk, int head_off, int hstep, int ng,
                                           int n, int np, int stride, bf16* dst, int vec) {
    const int n8 = np >> 3, total = ng * KT * n8;
    for (int idx = threadIdx.x; idx < total; idx += NT) {
        const int d = (idx % n8) << 3, rk = idx / n8, key = rk % KT, cl = rk / KT;
        bf16* to = dst + ((size_t)cl * KT + key) * stride + d;
        const bool live = key < nk && d < n;
        const bf16* src = pool + (live ? rowoff[key] + head_off + cl * hstep + d : 0);
        if (vec) {
            cp_async16(smem_addr(to), src, live);
        } else {
            unsigned short tmp[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) tmp[e] = (live && d + e < n) ? __bfloat16_as_ushort(src[e]) : (unsigned short)0;
            *reinterpret_cast<uint4*>(to) = make_uint4(tmp[0] | ((uint32_t)tmp[1] << 16), tmp[2] | ((uint32_t)tmp[3] << 16),
                                                       tmp[4] | ((uint32_t)tmp[5] << 16), tmp[6] | ((uint32_t)tmp[7] << 16));
        }
    }
}

// ONE (second pass without a head mix, all keys in one share): no first pass at all; the running maximum rescales the
// sums tile by tile and the division by the softmax sum comes last.
template <int KT, int NDV, bool APPLY, bool TALK, bool ONE>
__global__ void __launch_bounds__(NT) mix_tc_kernel(MixArgs a) {
    extern __shared__ __align__(16) unsigned char smraw[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int H = a.d.heads, G = a.d.kv_heads, rep = H / G, dk = a.d.dk, dv = a.d.dv, QT = a.QT, chunk = a.d.chunk;
    const int b = blockIdx.y;
    const int seq_end = a.cu_q[b + 1];
    // the last query tiles of a prompt see the most keys: they start first
    const int q_beg = a.cu_q[b] + (int)(gridDim.x - 1 - blockIdx.x) * QT;
    if (q_beg >= seq_end) return;
    const int nq = min(QT, seq_end - q_beg);
    const int share = blockIdx.z % a.shares, gsel = blockIdx.z / a.shares;
    const int gc0 = gsel * a.gp, gc1 = min(G, gc0 + a.gp), ng = gc1 - gc0;
    const int hbeg = gc0 * rep, rows = ng * rep * QT;
    const int dkp = a.dkp, DS = dkp + 8, VS = NDV * 8 + 8, kvw = DS > VS ? DS : VS;
    constexpr int PSF = KT + 8;
    const int pipe = a.rag;      // 1: two tile buffers, copies run behind the products; 0: one buffer, copy then compute
    const TcLayout L = tc_layout(a.gp * rep * QT, DS, VS, a.gp, KT, H, APPLY, TALK, pipe ? 2 : 1);
    bf16* Qh = reinterpret_cast<bf16*>(smraw + L.qh);
    bf16* Ql = reinterpret_cast<bf16*>(smraw + L.ql);
    bf16* kvb = reinterpret_cast<bf16*>(smraw + L.kv);
    bf16* kvb2 = kvb + (pipe ? (size_t)a.gp * KT * kvw : 0);
    float* Pm = reinterpret_cast<float*>(smraw + L.p);
    float* talk_s = reinterpret_cast<float*>(smraw + L.talk);
    float* Mr = reinterpret_cast<float*>(smraw + L.m);
    float* Lr = reinterpret_cast<float*>(smraw + L.l);
    long long* rowoff = reinterpret_cast<long long*>(smraw + L.off);
    const int M = a.ix.M;
    const int p0 = a.ix.positions[q_beg], p1 = p0 + nq - 1;
    const int kmin = chunk > 0 ? (p0 / chunk) * chunk : 0;
    const int ntile = (p1 - kmin) / KT + 1;
    const int per = (ntile + a.shares - 1) / a.shares;
    const int t0 = share * per, t1 = min(ntile, t0 + per);
    const int slot = a.seq_slot[b];
    const bf16* pool = static_cast<const bf16*>(a.cache.pool);
    const int row_elems = G * (dk + dv), psz = a.cache.page_size;

    // queries as two bf16 terms, row (h - hbeg) * QT + i, zero padded
    for (int idx = tid; idx < rows * dkp; idx += NT) {
        const int row = idx / dkp, d = idx - row * dkp;
        const int h = hbeg + row / QT, i = row % QT;
        const float v = (i < nq && d < dk) ? a.q[(long long)(q_beg + i) * a.ldq + (long long)h * dk + d] : 0.f;
        const bf16 hi = __float2bfloat16(v);
        Qh[(size_t)row * DS + d] = hi;
        Ql[(size_t)row * DS + d] = __float2bfloat16(v - __bfloat162float(hi));
    }
    if (APPLY && !ONE) {
        if (TALK)
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
    auto tile_rows = [&](int tl, long long* ro) {     // cache row offsets of tile tl's keys (threads below KT)
        if (tid < KT) {
            const int j = kmin + tl * KT + tid;
            long long off = 0;
            if (j <= p1) {
                const int page = a.cache.page_table[(long long)slot * a.cache.max_pages + j / psz];
                off = ((long long)page * psz + j % psz) * row_elems;
            }
            ro[tid] = off;
        }
    };
    if (pipe && t0 < t1) tile_rows(t0, rowoff + (t0 & 1) * KT);
    __syncthreads();
    if (pipe && t0 < t1) {
        stage_rows<KT>(pool, rowoff + (t0 & 1) * KT, min(KT, p1 - (kmin + t0 * KT) + 1), gc0 * dk, dk, ng, dk, dkp, kvw,
                       APPLY ? kvb : ((t0 & 1) ? kvb2 : kvb), a.vec);
        cp_async_commit();
    }

    const int rb = warp * 16;
    const bool active = rb < rows;
    int hx[2], ix_[2], posx[2], lox[2];
    bool okx[2];
    float Mx[2] = {0.f, 0.f}, iLx[2] = {0.f, 0.f};
#pragma unroll
    for (int x = 0; x < 2; ++x) {
        const int r = active ? rb + g + 8 * x : 0;
        hx[x] = hbeg + r / QT, ix_[x] = r % QT;
        posx[x] = p0 + ix_[x];
        lox[x] = chunk > 0 ? (posx[x] / chunk) * chunk : 0;
        okx[x] = active && ix_[x] < nq;
        if (APPLY && !ONE && active) Mx[x] = Mr[r], iLx[x] = Lr[r];
    }
    const int cw = active ? (hbeg + rb / QT) / rep - gc0 : 0;   // the warp's key/value group among the CTA's
    float mrun[2] = {-INFINITY, -INFINITY}, lrun[2] = {0.f, 0.f};
    float O[NDV][4];
#pragma unroll
    for (int n = 0; n < NDV; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) O[n][e] = 0.f;
    const int lr = lane & 7, mat = lane >> 3;

    for (int tl = t0; tl < t1; ++tl) {
        const int kb = kmin + tl * KT;
        const int nk = min(KT, p1 - kb + 1);
        const long long* ro = rowoff + (pipe ? (tl & 1) * KT : 0);
        bf16* kcur = (!APPLY && pipe && (tl & 1)) ? kvb2 : kvb;
        bf16* vcur = kvb2;
        const bool more = tl + 1 < t1;
        const int nk_next = min(KT, p1 - (kb + KT) + 1);
        if (pipe) {
            if (more) tile_rows(tl + 1, rowoff + ((tl + 1) & 1) * KT);
        } else {
            __syncthreads();
            tile_rows(tl, rowoff);
            __syncthreads();
            stage_rows<KT>(pool, ro, nk, gc0 * dk, dk, ng, dk, dkp, kvw, kcur, a.vec);
            cp_async_commit();
        }
        cp_async_wait<0>();
        __syncthreads();   // this tile's keys are here; every warp is done with the tile before
        if (pipe) {        // behind the score products: this tile's values (second pass) or the next tile's keys (first)
            if (APPLY) {
                stage_rows<KT>(pool, ro, nk, G * dk + gc0 * dv, dv, ng, dv, NDV * 8, kvw, vcur, a.vec);
                cp_async_commit();
            } else if (more) {
                stage_rows<KT>(pool, rowoff + ((tl + 1) & 1) * KT, nk_next, gc0 * dk, dk, ng, dk, dkp, kvw,
                               ((tl + 1) & 1) ? kvb2 : kvb, a.vec);
                cp_async_commit();
            }
        }
        float s[KT / 8][4];
#pragma unroll
        for (int n = 0; n < KT / 8; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[n][e] = 0.f;
        if (active) {
            const bf16* kt = kcur + (size_t)cw * KT * kvw;
            const uint32_t qh_addr = smem_addr(Qh + (size_t)(rb + lr + (mat & 1) * 8) * DS + (mat >> 1) * 8);
            const uint32_t ql_addr = smem_addr(Ql + (size_t)(rb + lr + (mat & 1) * 8) * DS + (mat >> 1) * 8);
            const uint32_t k_addr = smem_addr(kt + (size_t)(lr + (mat >> 1) * 8) * kvw + (mat & 1) * 8);
            for (int ks = 0; ks < dkp; ks += 16) {
                uint32_t ah[4], al[4];
                ldsm_x4(qh_addr + ks * 2, ah);
                ldsm_x4(ql_addr + ks * 2, al);
#pragma unroll
                for (int n2 = 0; n2 < KT / 16; ++n2) {
                    uint32_t bq[4];
                    ldsm_x4(k_addr + (n2 * 16 * kvw + ks) * 2, bq);
                    mma_bf16(s[2 * n2], ah, bq[0], bq[1]);
                    mma_bf16(s[2 * n2 + 1], ah, bq[2], bq[3]);
                    mma_bf16(s[2 * n2], al, bq[0], bq[1]);
                    mma_bf16(s[2 * n2 + 1], al, bq[2], bq[3]);
                }
            }
            float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int n = 0; n < KT / 8; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int x = e >> 1, col = n * 8 + 2 * t + (e & 1), j = kb + col;
                    const bool ok = okx[x] && col < nk && j <= posx[x] && j >= lox[x];
                    float v = s[n][e] * a.d.scale;
                    if (a.dist_bias && ok) v += a.dist_bias[(long long)min(posx[x] - j, a.far) * H + hx[x]];
                    v = ok ? v : -INFINITY;
                    if (!APPLY || ONE) {
                        s[n][e] = v;
                        tmax[x] = fmaxf(tmax[x], v);
                    } else {
                        s[n][e] = ok ? expf(v - Mx[x]) * iLx[x] : 0.f;
                    }
                }
            if (!APPLY) {
#pragma unroll
                for (int x = 0; x < 2; ++x) {
                    tmax[x] = fmaxf(tmax[x], __shfl_xor_sync(0xffffffffu, tmax[x], 1));
                    tmax[x] = fmaxf(tmax[x], __shfl_xor_sync(0xffffffffu, tmax[x], 2));
                    const float mnew = fmaxf(mrun[x], tmax[x]);
                    float sum = 0.f;
                    if (mnew > -INFINITY) {
#pragma unroll
                        for (int n = 0; n < KT / 8; ++n) {
                            sum += s[n][2 * x] > -INFINITY ? expf(s[n][2 * x] - mnew) : 0.f;
                            sum += s[n][2 * x + 1] > -INFINITY ? expf(s[n][2 * x + 1] - mnew) : 0.f;
                        }
                    }
                    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
                    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
                    if (mnew > -INFINITY) {
                        const float keep = mrun[x] > -INFINITY ? expf(mrun[x] - mnew) : 0.f;
                        lrun[x] = lrun[x] * keep + sum;
                        mrun[x] = mnew;
                    }
                }
            } else if (ONE) {
#pragma unroll
                for (int x = 0; x < 2; ++x) {
                    tmax[x] = fmaxf(tmax[x], __shfl_xor_sync(0xffffffffu, tmax[x], 1));
                    tmax[x] = fmaxf(tmax[x], __shfl_xor_sync(0xffffffffu, tmax[x], 2));
                    const float mnew = fmaxf(mrun[x], tmax[x]);
                    const float keep = (mrun[x] > -INFINITY && mnew > -INFINITY) ? expf(mrun[x] - mnew) : 0.f;
                    float sum = 0.f;      // this thread's part of the row's sum; the quad's parts are added at the end
#pragma unroll
                    for (int n = 0; n < KT / 8; ++n) {
                        const float w0 = s[n][2 * x] > -INFINITY ? expf(s[n][2 * x] - mnew) : 0.f;
                        const float w1 = s[n][2 * x + 1] > -INFINITY ? expf(s[n][2 * x + 1] - mnew) : 0.f;
                        s[n][2 * x] = w0, s[n][2 * x + 1] = w1;
                        sum += w0 + w1;
                    }
                    lrun[x] = lrun[x] * keep + sum;
                    mrun[x] = mnew;
#pragma unroll
                    for (int n = 0; n < NDV; ++n) O[n][2 * x] *= keep, O[n][2 * x + 1] *= keep;
                }
            } else if (TALK) {
#pragma unroll
                for (int n = 0; n < KT / 8; ++n) {
                    *reinterpret_cast<float2*>(Pm + (size_t)(rb + g) * PSF + n * 8 + 2 * t) = make_float2(s[n][0], s[n][1]);
                    *reinterpret_cast<float2*>(Pm + (size_t)(rb + g + 8) * PSF + n * 8 + 2 * t) = make_float2(s[n][2], s[n][3]);
                }
            }
        }
        if (!APPLY) continue;
        __syncthreads();   // every warp has read its keys; the weights of all heads are in shared memory
        if (pipe) {        // behind the mix and the value products: the next tile's keys
            if (more) {
                stage_rows<KT>(pool, rowoff + ((tl + 1) & 1) * KT, nk_next, gc0 * dk, dk, ng, dk, dkp, kvw, kvb, a.vec);
                cp_async_commit();
            }
        } else {
            stage_rows<KT>(pool, ro, nk, G * dk + gc0 * dv, dv, ng, dv, NDV * 8, kvw, vcur, a.vec);
            cp_async_commit();
        }
        if (TALK && active) {   // w'_h = sum_g talk[h][g] w_g, straight into this warp's fragment registers
#pragma unroll
            for (int n = 0; n < KT / 8; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) s[n][e] = 0.f;
            for (int gh = 0; gh < H; ++gh) {
                const float tk0 = talk_s[hx[0] * H + gh], tk1 = talk_s[hx[1] * H + gh];
                const float* pr0 = Pm + (size_t)(gh * QT + ix_[0]) * PSF + 2 * t;
                const float* pr1 = Pm + (size_t)(gh * QT + ix_[1]) * PSF + 2 * t;
#pragma unroll
                for (int n = 0; n < KT / 8; ++n) {
                    const float2 v0 = *reinterpret_cast<const float2*>(pr0 + n * 8);
                    const float2 v1 = *reinterpret_cast<const float2*>(pr1 + n * 8);
                    s[n][0] = fmaf(tk0, v0.x, s[n][0]);
                    s[n][1] = fmaf(tk0, v0.y, s[n][1]);
                    s[n][2] = fmaf(tk1, v1.x, s[n][2]);
                    s[n][3] = fmaf(tk1, v1.y, s[n][3]);
                }
            }
        }
        if (pipe && more)
            cp_async_wait<1>();     // the values; the next tile's keys stay in flight
        else
            cp_async_wait<0>();
        __syncthreads();
        if (active) {
            const bf16* vt = vcur + (size_t)cw * KT * kvw;
            const uint32_t v_addr = smem_addr(vt + (size_t)(lr + (mat & 1) * 8) * kvw + (mat >> 1) * 8);
#pragma unroll
            for (int j = 0; j < KT / 16; ++j) {
                uint32_t ph[4], pl[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const float w0 = s[2 * j + (u >> 1)][(u & 1) * 2], w1 = s[2 * j + (u >> 1)][(u & 1) * 2 + 1];
                    const bf16 h0 = __float2bfloat16(w0), h1 = __float2bfloat16(w1);
                    ph[u] = (uint32_t)__bfloat16_as_ushort(h0) | ((uint32_t)__bfloat16_as_ushort(h1) << 16);
                    pl[u] = pack_bf16(w0 - __bfloat162float(h0), w1 - __bfloat162float(h1));
                }
#pragma unroll
                for (int n = 0; n < NDV; n += 2) {
                    uint32_t bv[4];
                    ldsm_x4_t(v_addr + (j * 16 * kvw + n * 8) * 2, bv);
                    mma_bf16(O[n], ph, bv[0], bv[1]);
                    mma_bf16(O[n + 1], ph, bv[2], bv[3]);
                    mma_bf16(O[n], pl, bv[0], bv[1]);
                    mma_bf16(O[n + 1], pl, bv[2], bv[3]);
                }
            }
        }
    }

    if (!active) return;
    if (!APPLY) {
        if (t == 0) {
#pragma unroll
            for (int x = 0; x < 2; ++x) {
                if (!okx[x]) continue;
                const long long at = (long long)(q_beg + ix_[x]) * H + hx[x];
                a.stats[(long long)share * M * H + at] = mrun[x];
                a.stats[(long long)(a.shares + share) * M * H + at] = lrun[x];
            }
        }
        return;
    }
    if (ONE) {
#pragma unroll
        for (int x = 0; x < 2; ++x) {
            float l = lrun[x];
            l += __shfl_xor_sync(0xffffffffu, l, 1);
            l += __shfl_xor_sync(0xffffffffu, l, 2);
            const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
            for (int n = 0; n < NDV; ++n) O[n][2 * x] *= inv, O[n][2 * x + 1] *= inv;
        }
    }
#pragma unroll
    for (int x = 0; x < 2; ++x) {
        if (!okx[x]) continue;
        const int m = q_beg + ix_[x], h = hx[x];
        float gate = 1.f;
        if (a.shares == 1 && a.gate) gate = 1.f / (1.f + expf(-a.gate[(long long)m * a.ldg + h]));
#pragma unroll
        for (int n = 0; n < NDV; ++n)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int col = n * 8 + 2 * t + e;
                if (col >= dv) continue;
                const float v = O[n][2 * x + e];
                if (a.shares == 1)
                    stx(a.out, (long long)m * a.ldo + (long long)h * dv + col, a.of32, v * gate);
                else
                    a.part[((long long)share * M + m) * H * dv + (long long)h * dv + col] = v;
            }
    }
}

template <int KT, int NDV, bool APPLY, bool TALK, bool ONE>
int launch_tc(const MixArgs& a, dim3 grid, size_t smem, cudaStream_t stream) {
    static PerDeviceOnce once;
    if (once.need())
        ASD_CUDA(cudaFuncSetAttribute(mix_tc_kernel<KT, NDV, APPLY, TALK, ONE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      220 * 1024));
    mix_tc_kernel<KT, NDV, APPLY, TALK, ONE><<<grid, NT, smem, stream>>>(a);
    count_launch(1);
    ASD_CUDA(cudaGetLastError());
    return 0;
}

template <int KT, int NDV>
int launch_apply(const MixArgs& a, bool one, dim3 grid, size_t smem, cudaStream_t stream) {
    if (a.talk) return launch_tc<KT, NDV, true, true, false>(a, grid, smem, stream);
    return one ? launch_tc<KT, NDV, true, false, true>(a, grid, smem, stream)
               : launch_tc<KT, NDV, true, false, false>(a, grid, smem, stream);
}

template <int KT>
int launch_passes(const MixArgs& a, bool one, int ndv, dim3 grid, size_t smem_stats, size_t smem_apply, cudaStream_t stream) {
    if (!one && launch_tc<KT, 4, false, false, false>(a, grid, smem_stats, stream)) return -1;
    return ndv == 4 ? launch_apply<KT, 4>(a, one, grid, smem_apply, stream)
                    : (ndv == 8 ? launch_apply<KT, 8>(a, one, grid, smem_apply, stream)
                                : launch_apply<KT, 16>(a, one, grid, smem_apply, stream));
}

}  // namespace

int launch_mix_attention_tc(MixArgs a, int nseq, int max_qlen, int max_kv_len, const MixWork& ws, cudaStream_t stream) {
    const int H = a.d.heads, G = a.d.kv_heads, rep = H / G, dk = a.d.dk, dv = a.d.dv;
    if (a.cache.f32 || dv > 128 || max_qlen < 8 || (reinterpret_cast<uintptr_t>(a.cache.pool) & 15)) return 1;
    const bool talk = a.talk != nullptr;
    const int ndv = dv <= 32 ? 4 : (dv <= 64 ? 8 : 16);
    const int dkp = (dk + 15) & ~15, DS = dkp + 8, VS = ndv * 8 + 8;
    // queries per tile and key/value groups per CTA: rows = groups * rep * QT <= 128, a multiple of 16, and every block of
    // 16 rows inside one key/value group
    int QT = 0, gp = 0, KT = 0, pipe = 0;
    size_t smem_apply = 0;
    for (int qt = 32; qt >= 2 && !QT; qt >>= 1) {
        if (qt > 16 && max_qlen < 24) continue;
        if (qt > 8 && max_qlen < 12 && qt > 8) continue;
        const int g = talk ? G : std::min(G, 128 / std::max(1, rep * qt));
        if (g < 1 || g * rep * qt > 128 || (g * rep * qt) % 16) continue;
        if (!(qt % 16 == 0 || (16 % qt == 0 && rep % (16 / qt) == 0))) continue;
        for (int nbuf : {2, 1}) {
            for (int kt : {64, 32}) {
                const size_t sm = (size_t)tc_layout(g * rep * qt, DS, VS, g, kt, H, true, talk, nbuf).total;
                if (sm <= 200 * 1024) {
                    QT = qt, gp = g, KT = kt, smem_apply = sm, pipe = nbuf == 2;
                    break;
                }
            }
            if (QT) break;
        }
    }
    if (!QT) return 1;
    a.QT = QT, a.gp = gp, a.dkp = dkp, a.dvp = ndv * 8, a.rag = pipe;
    a.vec = (dk % 8 == 0 && dv % 8 == 0) ? 1 : 0;
    const int tiles = (max_qlen + QT - 1) / QT, ngroups = (G + gp - 1) / gp;
    int shares = 1;
    const long long base = (long long)tiles * nseq * ngroups;
    const int key_tiles = (max_kv_len + KT - 1) / KT;
    if (base < 148 && ws.part) {
        shares = (int)std::min<long long>((296 + base - 1) / base, (long long)std::max(1, key_tiles / 2));
        shares = std::min(shares, 32);
        while (shares > 1 && ((long long)shares * a.ix.M * H * dv > ws.part_elems ||
                              (long long)2 * shares * a.ix.M * H > ws.stats_elems))
            --shares;
    }
    if (!ws.stats || (long long)2 * shares * a.ix.M * H > ws.stats_elems) return 1;
    a.shares = shares;
    const size_t smem_stats = (size_t)tc_layout(gp * rep * QT, DS, VS, gp, KT, H, false, false, pipe ? 2 : 1).total;
    const dim3 grid(tiles, nseq, shares * ngroups);
    const bool one = !talk && shares == 1;      // no mix across heads and one share: one pass with a running maximum
    const int rc = KT == 64 ? launch_passes<64>(a, one, ndv, grid, smem_stats, smem_apply, stream)
                            : launch_passes<32>(a, one, ndv, grid, smem_stats, smem_apply, stream);
    if (rc) return -1;
    if (shares > 1 && launch_mix_merge(a, stream)) return -1;
    return 0;
}

}  // namespace asd
