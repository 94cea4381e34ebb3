// Row kernels of sandwich-normed layers: scaled embedding, the close of a sublayer fused with the norm that follows
// (residual sum, norm after the sublayer, norm before the next one, optionally the concatenation a pass entry reads),
// plain / offset RMS norm of a slice of a row, the normalised cubic polynomial of a feed-forward row, the tanh cap of
// the logits; the normed embedding and the elementwise activations of plain and gated feed-forwards.  A norm may split
// its row into equal consecutive groups, each divided by its own root mean square.  One CTA per row; sums of squares,
// the residual stream and every norm are fp32 whatever the engine's type.
#include <cuda_bf16.h>

#include "asd_internal.h"
#include "blocks.h"
#include "elem.cuh"

namespace asd {

namespace {

inline int row_threads(int D) { return D >= 2048 ? 512 : (D >= 1024 ? 256 : (D >= 256 ? 128 : 64)); }

__global__ void embed_scaled_kernel(SeqIndex ix, const void* embed, int wf32, float scale, float* x0, float* x, int D) {
    const int m = blockIdx.x;
    const long long src = (long long)ix.tokens[m] * D, dst = (long long)m * D;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        const float v = ldx(embed, src + d, wf32) * scale;
        x0[dst + d] = v;
        if (x) x[dst + d] = v;
    }
}

constexpr int MAX_NORM_GROUPS = 64;   // parts a grouped norm may split a row into

// dynamic shared memory: D floats (the row being built) + 33 for the block sums + MAX_NORM_GROUPS group factors
__global__ void row_close_kernel(RowClose c) {
    extern __shared__ float sm[];
    float* row = sm;
    float* red = sm + c.D;
    float* gs = red + 33;
    const int m = blockIdx.x, D = c.D, G = c.groups, Dg = D / G;
    const long long base = (long long)m * D;
    const long long in_base = c.rows ? (long long)c.rows[m] * D : base;
    const float off = c.plain_w ? 0.f : 1.f;
    float post = 1.f;
    if (c.y && c.post_w) {
        float ss = 0.f;
        for (int d = threadIdx.x; d < D; d += blockDim.x) {
            const float v = c.y[base + d];
            ss += v * v;
        }
        post = 1.f / sqrtf(block_sum(ss, red) / (float)D + c.eps);
    }
#pragma unroll 4
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float v = c.x_in ? c.x_in[in_base + d] : 0.f;
        if (c.y) v += c.post_w ? c.y[base + d] * post * (off + c.post_w[d]) : c.y[base + d];
        for (int k = 0; k < c.top; ++k)     // routed experts' results in choice order
            v = fmaf(c.gate[(long long)m * c.top + k], c.expert_out[(long long)c.slot_of[(long long)m * c.top + k] * D + d], v);
        if (c.bias) v += c.bias[d];
        row[d] = v;
        if (c.x_out) c.x_out[base + d] = v;
    }
    if (c.next_w) {
        __syncthreads();
        for (int g = 0; g < G; ++g) {
            float ss = 0.f;
            for (int d = g * Dg + threadIdx.x; d < (g + 1) * Dg; d += blockDim.x) ss += row[d] * row[d];
            const float t = block_sum(ss, red);
            if (threadIdx.x == 0) gs[g] = 1.f / sqrtf(t / (float)Dg + c.eps);
        }
        __syncthreads();
        for (int d = threadIdx.x; d < D; d += blockDim.x)
            stx(c.hn, base + d, c.hn_f32, row[d] * gs[d / Dg] * (off + c.next_w[d]));
    } else if (c.cat) {
        for (int d = threadIdx.x; d < D; d += blockDim.x) {
            stx(c.hn, 2 * base + d, c.hn_f32, row[d]);
            stx(c.hn, 2 * base + D + d, c.hn_f32, c.cat[base + d]);
        }
    }
}

// x[m] = group_norm(embed[token]) * w, fp32 (dynamic shared memory as row_close_kernel)
__global__ void embed_normed_kernel(SeqIndex ix, const void* embed, int wf32, const float* w, int groups, float eps, float* x,
                                    int D) {
    extern __shared__ float sm[];
    float* row = sm;
    float* red = sm + D;
    float* gs = red + 33;
    const int m = blockIdx.x, Dg = D / groups;
    const long long src = (long long)ix.tokens[m] * D, dst = (long long)m * D;
    for (int d = threadIdx.x; d < D; d += blockDim.x) row[d] = ldx(embed, src + d, wf32);
    __syncthreads();
    for (int g = 0; g < groups; ++g) {
        float ss = 0.f;
        for (int d = g * Dg + threadIdx.x; d < (g + 1) * Dg; d += blockDim.x) ss += row[d] * row[d];
        const float t = block_sum(ss, red);
        if (threadIdx.x == 0) gs[g] = 1.f / sqrtf(t / (float)Dg + eps);
    }
    __syncthreads();
    for (int d = threadIdx.x; d < D; d += blockDim.x) x[dst + d] = row[d] * gs[d / Dg] * w[d];
}

__device__ __forceinline__ float gelu_tanh_f(float z) {
    return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// out[r][f] = gelu_tanh(z[r][f]) (mode 0, z rows of F floats) or silu(z[r][f]) * z[r][F + f] (mode 1, rows of 2 F)
// mode 2: relu(z[r][f])^2.  bias (optional) is added to z first: [F], or [2 F] in mode 1.
__global__ void ff_act_kernel(const float* z, void* out, int of32, long long n, int F, int mode, const float* bias) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    if (mode != 1) {
        float v = z[i];
        if (bias) v += bias[(int)(i % F)];
        if (mode == 0) {
            stx(out, i, of32, gelu_tanh_f(v));
        } else {
            v = fmaxf(v, 0.f);
            stx(out, i, of32, v * v);
        }
    } else {
        const long long r = i / F;
        const int f = (int)(i - r * F);
        float g = z[r * 2 * F + f], u = z[r * 2 * F + F + f];
        if (bias) g += bias[f], u += bias[F + f];
        stx(out, i, of32, g / (1.f + expf(-g)) * u);
    }
}

__global__ void rms_rows_kernel(const float* in, long long ld_in, const float* w, int plus_one, float eps, void* out,
                                int of32, long long ld_out, int n) {
    __shared__ float red[33];
    const float* src = in + (long long)blockIdx.x * ld_in;
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) ss += src[i] * src[i];
    const float r = 1.f / sqrtf(block_sum(ss, red) / (float)n + eps);
    for (int i = threadIdx.x; i < n; i += blockDim.x)
        stx(out, (long long)blockIdx.x * ld_out + i, of32, src[i] * r * (plus_one ? 1.f + w[i] : w[i]));
}

// dynamic shared memory: the row (F floats, if it fits: `staged`) + 33 for the block sums
__global__ void polynorm_kernel(const float* z, const float* coeff, float eps, void* out, int of32, int F, int staged) {
    extern __shared__ float sm[];
    float* red = sm;
    float* row = sm + 33;
    const float* src = z + (long long)blockIdx.x * F;
    float s2 = 0.f, s4 = 0.f, s6 = 0.f;
    for (int i = threadIdx.x; i < F; i += blockDim.x) {
        const float v = src[i], v2 = v * v, v3 = v2 * v;
        if (staged) row[i] = v;
        s2 += v2;
        s4 += v2 * v2;
        s6 += v3 * v3;
    }
    s2 = block_sum(s2, red);
    s4 = block_sum(s4, red);
    s6 = block_sum(s6, red);
    const float inv = 1.f / (float)F;
    const float a = coeff[0] / sqrtf(s2 * inv + eps), b = coeff[1] / sqrtf(s4 * inv + eps),
                c = coeff[2] / sqrtf(s6 * inv + eps), e = coeff[3];
    for (int i = threadIdx.x; i < F; i += blockDim.x) {
        const float v = staged ? row[i] : src[i], v2 = v * v;
        stx(out, (long long)blockIdx.x * F + i, of32, a * v + b * v2 + c * (v2 * v) + e);
    }
}

__global__ void softcap_kernel(float* logits, long long ld, int V, float cap) {
    float* row = logits + (long long)blockIdx.x * ld;
    const int i = blockIdx.y * blockDim.x + threadIdx.x;
    if (i < V) row[i] = cap * tanhf(row[i] / cap);
}

}  // namespace

int launch_embed_scaled(const SeqIndex& ix, const void* embed, int wf32, float scale, float* x0, float* x, int D,
                        cudaStream_t stream) {
    if (ix.M <= 0) return 0;
    embed_scaled_kernel<<<ix.M, row_threads(D), 0, stream>>>(ix, embed, wf32, scale, x0, x, D);
    count_launch(1);
    ASD_CUDA(cudaGetLastError());
    return 0;
}

int launch_row_close(const RowClose& c, cudaStream_t stream) {
    if (c.M <= 0) return 0;
    if (c.D <= 0 || ((c.next_w || c.cat) && !c.hn)) return set_error("row_close: bad arguments");
    if (c.groups <= 0 || c.groups > MAX_NORM_GROUPS || c.D % c.groups)
        return set_error("row_close: %d norm groups do not divide width %d (at most %d)", c.groups, c.D, MAX_NORM_GROUPS);
    if (c.top > 0 && (!c.expert_out || !c.slot_of || !c.gate)) return set_error("row_close: expert results missing");
    const size_t smem = (size_t)(c.D + 33 + MAX_NORM_GROUPS) * sizeof(float);
    if (smem > 200 * 1024) return set_error("row_close: width %d does not fit shared memory", c.D);
    static PerDeviceOnce once;
    if (once.need()) ASD_CUDA(cudaFuncSetAttribute(row_close_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
    row_close_kernel<<<c.M, row_threads(c.D), smem, stream>>>(c);
    count_launch(1);
    ASD_CUDA(cudaGetLastError());
    return 0;
}

int launch_embed_normed(const SeqIndex& ix, const void* embed, int wf32, const float* w, int groups, float eps, float* x,
                        int D, cudaStream_t stream) {
    if (ix.M <= 0) return 0;
    if (groups <= 0 || groups > MAX_NORM_GROUPS || D % groups)
        return set_error("embed_normed: %d norm groups do not divide width %d (at most %d)", groups, D, MAX_NORM_GROUPS);
    const size_t smem = (size_t)(D + 33 + MAX_NORM_GROUPS) * sizeof(float);
    if (smem > 200 * 1024) return set_error("embed_normed: width %d does not fit shared memory", D);
    static PerDeviceOnce once;
    if (once.need()) ASD_CUDA(cudaFuncSetAttribute(embed_normed_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
    embed_normed_kernel<<<ix.M, row_threads(D), smem, stream>>>(ix, embed, wf32, w, groups, eps, x, D);
    count_launch(1);
    ASD_CUDA(cudaGetLastError());
    return 0;
}

int launch_ff_act(const float* z, void* out, int of32, long long rows, int F, int gated, cudaStream_t stream,
                  const float* bias) {
    const long long n = rows * F;
    if (n <= 0) return 0;
    const long long blocks = (n + 255) / 256;
    if (blocks > 0x7fffffffLL) return set_error("ff_act: too many elements");
    ff_act_kernel<<<(unsigned)blocks, 256, 0, stream>>>(z, out, of32, n, F, gated, bias);
    count_launch(1);
    ASD_CUDA(cudaGetLastError());
    return 0;
}

int launch_rms_rows(const float* in, long long ld_in, const float* w, int plus_one, float eps, void* out, int of32,
                    long long ld_out, int M, int n, cudaStream_t stream) {
    if (M <= 0 || n <= 0) return 0;
    rms_rows_kernel<<<M, row_threads(n), 0, stream>>>(in, ld_in, w, plus_one, eps, out, of32, ld_out, n);
    count_launch(1);
    ASD_CUDA(cudaGetLastError());
    return 0;
}

int launch_polynorm(const float* z, const float* coeff, float eps, void* out, int of32, int M, int F, cudaStream_t stream) {
    if (M <= 0 || F <= 0) return 0;
    const int staged = (size_t)F * sizeof(float) <= 96 * 1024;
    const size_t smem = (33 + (staged ? (size_t)F : 0)) * sizeof(float);
    static PerDeviceOnce once;
    if (once.need()) ASD_CUDA(cudaFuncSetAttribute(polynorm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
    polynorm_kernel<<<M, row_threads(F), smem, stream>>>(z, coeff, eps, out, of32, F, staged);
    count_launch(1);
    ASD_CUDA(cudaGetLastError());
    return 0;
}

int launch_softcap(float* logits, long long ld, int n, int V, float cap, cudaStream_t stream) {
    if (n <= 0 || V <= 0 || !(cap > 0.f)) return 0;
    dim3 grid(n, (V + 255) / 256);
    softcap_kernel<<<grid, 256, 0, stream>>>(logits, ld, V, cap);
    count_launch(1);
    ASD_CUDA(cudaGetLastError());
    return 0;
}

}  // namespace asd
