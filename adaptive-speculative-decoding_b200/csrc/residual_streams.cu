// Several residual streams per token (hyper-connections).  A token's row holds S copies of the model width, fp32
// [M][S][D].  A sublayer reads the weighted sum u = sum_s read[s] x_s; its result y returns to all streams at once,
//   x_t <- sum_s mix[s][t] x_s + write[t] * y,
// computed from the old streams.  One CTA owns a row: it updates the streams in place (every element's S old values
// are in registers before any is written), forms the next sublayer's u on the way, and norms it.  Everything is fp32.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "asd_internal.h"
#include "blocks.h"
#include "elem.cuh"

namespace asd {

constexpr int MAX_STREAMS = 16;

__global__ void embed_streams_kernel(SeqIndex ix, const void* embed, const void* pos_table, int wf32, float scale, float* xs,
                                     int S, int D) {
    const int m = blockIdx.x;
    const long long src = (long long)ix.tokens[m] * D, psrc = (long long)ix.positions[m] * D;
    float* dst = xs + (long long)m * S * D;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float v = ldx(embed, src + d, wf32) * scale;
        if (pos_table) v += ldx(pos_table, psrc + d, wf32);
        for (int s = 0; s < S; ++s) dst[(long long)s * D + d] = v;
    }
}

// dynamic shared memory: D floats (u) + 33 (block sums) + S * S + 2 S (the sublayer's small weights)
template <int S_>
__global__ void stream_close_kernel(StreamClose c) {
    extern __shared__ float sm[];
    const int S = S_ > 0 ? S_ : c.S, D = c.D;
    float* u = sm;
    float* red = sm + D;
    float* wmix = red + 33;
    float* wwrite = wmix + S * S;
    float* wread = wwrite + S;
    const int m = blockIdx.x;
    const long long src_row = c.rows ? (long long)c.rows[m] : (long long)m;
    float* xrow = c.xs + src_row * S * D;
    const bool update = c.y != nullptr && c.rows == nullptr;
    const bool reads = c.read != nullptr || c.want_sum;
    for (int i = threadIdx.x; i < S * S; i += blockDim.x) wmix[i] = c.mix ? c.mix[i] : ((i / S) == (i % S) ? 1.f : 0.f);
    for (int i = threadIdx.x; i < S; i += blockDim.x) {
        wwrite[i] = c.write ? c.write[i] : 1.f;
        wread[i] = c.read ? c.read[i] : 1.f;
    }
    __syncthreads();
    float ss = 0.f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float xo[S_ > 0 ? S_ : MAX_STREAMS];
#pragma unroll
        for (int s = 0; s < (S_ > 0 ? S_ : MAX_STREAMS); ++s)
            if (s < S) xo[s] = xrow[(long long)s * D + d];
        float acc = 0.f;
        if (update) {
            float yv = c.y[(long long)m * D + d];
            if (c.y_bias) yv += c.y_bias[d];
#pragma unroll
            for (int t = 0; t < (S_ > 0 ? S_ : MAX_STREAMS); ++t) {
                if (t >= S) break;
                float v = 0.f;
#pragma unroll
                for (int s = 0; s < (S_ > 0 ? S_ : MAX_STREAMS); ++s)
                    if (s < S) v = fmaf(wmix[s * S + t], xo[s], v);
                v = fmaf(wwrite[t], yv, v);
                xrow[(long long)t * D + d] = v;
                acc = fmaf(wread[t], v, acc);
            }
        } else {
#pragma unroll
            for (int s = 0; s < (S_ > 0 ? S_ : MAX_STREAMS); ++s)
                if (s < S) acc = fmaf(wread[s], xo[s], acc);
        }
        if (reads) {
            u[d] = acc;
            ss += acc * acc;
            if (c.u_out) c.u_out[(long long)m * D + d] = acc;
        }
    }
    if (!reads || !c.next_w) return;
    const float r = 1.f / sqrtf(block_sum(ss, red) / (float)D + c.eps);
    for (int d = threadIdx.x; d < D; d += blockDim.x) stx(c.hn, (long long)m * D + d, c.hn_f32, u[d] * r * c.next_w[d]);
}

static inline int stream_threads(int D) { return D >= 2048 ? 512 : (D >= 1024 ? 256 : (D >= 256 ? 128 : 64)); }

int launch_embed_streams(const SeqIndex& ix, const void* embed, const void* pos_table, int wf32, float scale, float* xs,
                         int S, int D, cudaStream_t stream) {
    if (ix.M <= 0) return 0;
    if (S <= 0 || D <= 0) return set_error("embed_streams: bad sizes");
    embed_streams_kernel<<<ix.M, stream_threads(D), 0, stream>>>(ix, embed, pos_table, wf32, scale, xs, S, D);
    count_launch(1);
    ASD_CUDA(cudaGetLastError());
    return 0;
}

template <int S_>
static int launch_close(const StreamClose& c, size_t smem, cudaStream_t stream) {
    static PerDeviceOnce once;
    if (once.need())
        ASD_CUDA(cudaFuncSetAttribute(stream_close_kernel<S_>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
    stream_close_kernel<S_><<<c.M, stream_threads(c.D), smem, stream>>>(c);
    count_launch(1);
    ASD_CUDA(cudaGetLastError());
    return 0;
}

int launch_stream_close(const StreamClose& c, cudaStream_t stream) {
    if (c.M <= 0) return 0;
    if (c.D <= 0 || c.S <= 0 || c.S > MAX_STREAMS || !c.xs)
        return set_error("stream_close: bad sizes (%d streams, at most %d)", c.S, MAX_STREAMS);
    if (c.next_w && !c.hn) return set_error("stream_close: no output for the normed row");
    const size_t smem = (size_t)(c.D + 33 + c.S * c.S + 2 * c.S) * sizeof(float);
    if (smem > 200 * 1024) return set_error("stream_close: width %d does not fit shared memory", c.D);
    switch (c.S) {
        case 1: return launch_close<1>(c, smem, stream);
        case 2: return launch_close<2>(c, smem, stream);
        case 3: return launch_close<3>(c, smem, stream);
        case 4: return launch_close<4>(c, smem, stream);
        case 6: return launch_close<6>(c, smem, stream);
        case 8: return launch_close<8>(c, smem, stream);
        default: return launch_close<0>(c, smem, stream);
    }
}

}  // namespace asd
