// Internal declarations shared by the kernels of the mixed-weights attention (mixed_attention.cu: CUDA cores, any sizes,
// both element types; mixed_attention_tc.cu: prompts of a bf16 engine on the tensor cores; steps of few tokens).
#pragma once
#include <cuda_runtime.h>

#include "blocks.h"

namespace asd {

struct MixArgs {
    SeqIndex ix;
    const int* cu_q;
    const int* seq_slot;
    const float* q;
    long long ldq;
    MixDims d;
    const float* dist_bias;
    int far;
    const float* talk;
    const float* gate;
    long long ldg;
    PagedRows cache;
    void* out;
    int of32;
    long long ldo;
    float* stats;      // [2][shares][M][heads]: maximum, then sum of exponentials, of every key share
    float* part;       // [shares][M][heads * dv]
    float* scores;     // steps of few tokens: [M][heads][score_ld] scaled, biased scores of the visible keys
    long long score_ld;
    int QT, shares, gp, rag, dkp, dvp, vec;
};

// Prompts and portions of a bf16 engine on the tensor cores (mma.sync, fp32 operands as two bf16 terms).  Returns 1 if
// these sizes are not taken (the caller then runs the CUDA-core kernels), 0 after the launches, -1 on an error.
int launch_mix_attention_tc(MixArgs a, int nseq, int max_qlen, int max_kv_len, const MixWork& ws, cudaStream_t stream);
// Steps of one token per sequence: scores once (kept in the workspace), then weights, mix and values.  Same returns.
int launch_mix_attention_decode(MixArgs a, int nseq, int max_kv_len, const MixWork& ws, cudaStream_t stream);
// sums the key shares' partial results in index order, applies the gates, writes the engine's element type
int launch_mix_merge(const MixArgs& a, cudaStream_t stream);

}  // namespace asd
