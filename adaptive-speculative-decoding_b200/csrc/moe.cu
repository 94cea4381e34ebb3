// Mixture-of-experts routing: fp32 softmax over all experts, the `top` largest probabilities kept as gates (as they
// are, or divided by their sum, which is the softmax over the chosen logits alone), then the (token, choice) pairs grouped by expert so that each expert's rows are contiguous
// for the grouped linear layers.  Which slot inside an expert's group a pair gets does not matter for the result: every
// slot is computed on its own and a token's choices are summed in choice order by the layer close.
#include <cuda_runtime.h>
#include <math.h>

#include "asd_internal.h"
#include "blocks.h"
#include "elem.cuh"

namespace asd {

namespace {

// one warp per token; probs of the token live in shared memory (E floats per warp).  With x != nullptr the warp first
// computes the token's router logits itself, z[e] = sum_d x[m][d] * wr[e][d] in fp32 (lane-strided partial sums in
// increasing d, then the fixed warp tree: the same for a token whatever else is in the batch), eight experts per pass
// over the row.
__global__ void moe_route_kernel(const float* logits, const void* x, int xf32, const void* wr, int wf32, int D, float* z_out,
                                 int M, int E, int top, int* expert_of, float* gate, int* counts, const float* bias,
                                 int renorm) {
    extern __shared__ float sm[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m = blockIdx.x * (blockDim.x >> 5) + warp;
    if (m >= M) return;
    float* pr = sm + (size_t)warp * E;
    float* zs = sm + (size_t)(blockDim.x >> 5) * E + (size_t)warp * E;
    if (x) {
        for (int e0 = 0; e0 < E; e0 += 8) {
            float acc[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = 0.f;
            for (int d = lane; d < D; d += 32) {
                const float xv = ldx(x, (long long)m * D + d, xf32);
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    if (e0 + j < E) acc[j] = fmaf(xv, ldx(wr, (long long)(e0 + j) * D + d, wf32), acc[j]);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float v = warp_sum(acc[j]);
                if (lane == 0 && e0 + j < E) {
                    const float zb = bias ? v + bias[e0 + j] : v;
                    zs[e0 + j] = zb;
                    if (z_out) z_out[(long long)m * E + e0 + j] = zb;
                }
            }
        }
        __syncwarp();
    }
    const float* z = x ? zs : logits + (long long)m * E;
    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, z[e]);
    mx = warp_max(mx);
    float s = 0.f;
    for (int e = lane; e < E; e += 32) {
        const float v = expf(z[e] - mx);
        pr[e] = v;
        s += v;
    }
    s = warp_sum(s);
    const float inv = 1.f / s;
    float chosen = 0.f;
    __syncwarp();
    for (int k = 0; k < top; ++k) {
        float best = -1.f;
        int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = pr[e];
            if (v > best) {        // increasing e per lane: the first maximum wins
                best = v;
                bi = e;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ob > best || (ob == best && oi < bi)) {
                best = ob;
                bi = oi;
            }
        }
        if (lane == 0) {
            expert_of[(long long)m * top + k] = bi;
            gate[(long long)m * top + k] = best * inv;
            chosen += best;
            atomicAdd(&counts[bi], 1);
            pr[bi] = -2.f;         // taken
        }
        __syncwarp();
    }
    if (renorm && lane == 0) {   // gates over the chosen alone: e^(z - max) / sum of the chosen e^(z - max)
        const float r = 1.f / (chosen * inv);
        for (int k = 0; k < top; ++k) gate[(long long)m * top + k] *= r;
    }
}

// Few tokens (M * top <= 4096): choice, group sizes, offsets and scatter in ONE CTA with shared-memory counters, so that a
// decode step spends two launches on routing (logits, then this) instead of five.
__global__ void __launch_bounds__(256) moe_route_small_kernel(const float* logits, int M, int E, int top, int* expert_of,
                                                              float* gate, int* group_off, int* sorted_tok, int* slot_of,
                                                              int renorm) {
    extern __shared__ float sm[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    int* cnt = reinterpret_cast<int*>(sm + (size_t)nw * E);     // [E] group sizes, then fill counters
    int* off = cnt + E;                                          // [E + 1]
    for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
    __syncthreads();
    float* pr = sm + (size_t)warp * E;
    for (int m = warp; m < M; m += nw) {
        const float* z = logits + (long long)m * E;
        float mx = -INFINITY;
        for (int e = lane; e < E; e += 32) mx = fmaxf(mx, z[e]);
        mx = warp_max(mx);
        float s = 0.f;
        for (int e = lane; e < E; e += 32) {
            const float v = expf(z[e] - mx);
            pr[e] = v;
            s += v;
        }
        s = warp_sum(s);
        const float inv = 1.f / s;
        float chosen = 0.f;
        __syncwarp();
        for (int k = 0; k < top; ++k) {
            float best = -1.f;
            int bi = 0x7fffffff;
            for (int e = lane; e < E; e += 32) {
                const float v = pr[e];
                if (v > best) {
                    best = v;
                    bi = e;
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (ob > best || (ob == best && oi < bi)) {
                    best = ob;
                    bi = oi;
                }
            }
            if (lane == 0) {
                expert_of[(long long)m * top + k] = bi;
                gate[(long long)m * top + k] = best * inv;
                chosen += best;
                atomicAdd(&cnt[bi], 1);
                pr[bi] = -2.f;
            }
            __syncwarp();
        }
        if (renorm && lane == 0) {
            const float r = 1.f / (chosen * inv);
            for (int k = 0; k < top; ++k) gate[(long long)m * top + k] *= r;
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int o = 0;
        for (int e = 0; e < E; ++e) {
            off[e] = o;
            group_off[e] = o;
            o += cnt[e];
            cnt[e] = 0;
        }
        off[E] = o;
        group_off[E] = o;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < M * top; i += blockDim.x) {
        const int e = expert_of[i];
        const int slot = off[e] + atomicAdd(&cnt[e], 1);
        sorted_tok[slot] = i / top;
        slot_of[i] = slot;
    }
}

// router logits, one CTA per token: z[m][e] = sum_d x[m][d] * wr[e][d] in fp32.  Thread t sums d = t, t + 128, ... in
// increasing order, then the fixed warp tree and the warps in index order: a token's logits do not depend on the batch.
__global__ void __launch_bounds__(128) moe_logits_kernel(const void* x, int xf32, const void* wr, int wf32, int D, int E,
                                                         float* z_out, const float* bias) {
    __shared__ float red[4][8];
    const int m = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int e0 = 0; e0 < E; e0 += 8) {
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll 4
        for (int d = threadIdx.x; d < D; d += 128) {
            const float xv = ldx(x, (long long)m * D + d, xf32);
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (e0 + j < E) acc[j] = fmaf(xv, ldx(wr, (long long)(e0 + j) * D + d, wf32), acc[j]);
        }
        __syncthreads();
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float v = warp_sum(acc[j]);
            if (lane == 0) red[warp][j] = v;
        }
        __syncthreads();
        if (threadIdx.x < 8 && e0 + threadIdx.x < E)
            z_out[(long long)m * E + e0 + threadIdx.x] =
                (((red[0][threadIdx.x] + red[1][threadIdx.x]) + red[2][threadIdx.x]) + red[3][threadIdx.x]) +
                (bias ? bias[e0 + threadIdx.x] : 0.f);
    }
}

__global__ void moe_offsets_kernel(int* counters, int* group_off, int E) {
    if (threadIdx.x == 0) {
        int o = 0;
        for (int e = 0; e < E; ++e) {
            group_off[e] = o;
            o += counters[e];
            counters[E + e] = 0;   // fill counters of the scatter pass
        }
        group_off[E] = o;
    }
}

__global__ void moe_scatter_kernel(const int* expert_of, int n, int top, int E, const int* group_off, int* counters,
                                   int* sorted_tok, int* slot_of) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int e = expert_of[i];
    const int slot = group_off[e] + atomicAdd(&counters[E + e], 1);
    sorted_tok[slot] = i / top;
    slot_of[i] = slot;
}

}  // namespace

int launch_moe_route(const float* logits, const MoeRouterInput* in, int M, int E, int top, int* expert_of, float* gate,
                     int* counters, int* group_off, int* sorted_tok, int* slot_of, cudaStream_t stream) {
    if (M <= 0) return 0;
    if (E <= 0 || top <= 0 || top > E) return set_error("moe: need 0 < top <= experts (top %d, experts %d)", top, E);
    if ((size_t)E * 8 * sizeof(float) > 48 * 1024) return set_error("moe: more than 1536 experts");
    if (!logits && !in) return set_error("moe: neither logits nor router inputs");
    const int renorm = in ? in->renorm : 0;
    if (in && in->logits_out && (long long)M * top <= 4096 && (size_t)(8 * E + 2 * E + 1) * 4 <= 48 * 1024) {
        moe_logits_kernel<<<M, 128, 0, stream>>>(in->x, in->x_f32, in->w, in->w_f32, in->D, E, in->logits_out, in->bias);
        moe_route_small_kernel<<<1, 256, (size_t)(8 * E + 2 * E + 1) * sizeof(float), stream>>>(
            in->logits_out, M, E, top, expert_of, gate, group_off, sorted_tok, slot_of, in->renorm);
        count_launch(2);
        ASD_CUDA(cudaGetLastError());
        return 0;
    }
    ASD_CUDA(cudaMemsetAsync(counters, 0, sizeof(int) * E, stream));
    if (in && in->logits_out) {          // a CTA per token for the logits: few tokens still spread over the GPU
        moe_logits_kernel<<<M, 128, 0, stream>>>(in->x, in->x_f32, in->w, in->w_f32, in->D, E, in->logits_out, in->bias);
        count_launch(1);
        logits = in->logits_out;
        in = nullptr;
    }
    moe_route_kernel<<<(M + 3) / 4, 128, (size_t)E * 8 * sizeof(float), stream>>>(
        logits, in ? in->x : nullptr, in ? in->x_f32 : 0, in ? in->w : nullptr, in ? in->w_f32 : 0, in ? in->D : 0,
        nullptr, M, E, top, expert_of, gate, counters, in ? in->bias : nullptr, renorm);
    moe_offsets_kernel<<<1, 32, 0, stream>>>(counters, group_off, E);
    const int n = M * top;
    moe_scatter_kernel<<<(n + 255) / 256, 256, 0, stream>>>(expert_of, n, top, E, group_off, counters, sorted_tok, slot_of);
    count_launch(3);
    ASD_CUDA(cudaGetLastError());
    return 0;
}

}  // namespace asd
