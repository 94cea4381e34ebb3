// Mavipel family forward engine: one opaque handle per model.  asd_mavipel_forward runs, on the caller's stream and with
// no host synchronisation,
//   normed embedding -> for every layer execution [ (pass entry: + the pass's vector) grouped norm, mixer, residual,
//   grouped norm, feed-forward, residual ] -> final norm of the wanted rows, head.
// A layer's mixer is either the gated delta rule over short-convolved, unit-length queries and keys ("channel_delta"),
// or two mixers side by side on the same input ("parallel"): talking-heads window attention with a sink, and the
// generalised delta rule; their results are scaled and summed through one stacked output projection.  The feed-forward
// is a two-matrix gelu layer or routed gated experts plus a shared one.  Layers of a repeated span execute several times
// with the same weights and a cache or state per execution.  Every step is a building block of blocks.h that takes its
// sizes from the layer's configuration; dense bf16 projections go to the tcgen05 GEMMs when their shape fits (dense.h).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <string.h>

#include <algorithm>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/asd_b200.h"
#include "asd_internal.h"
#include "blocks.h"
#include "dense.h"
#include "prof.h"

struct asd_mavipel_engine {};

namespace asd {

enum MvType { MV_CHANNEL_DELTA = 0, MV_PARALLEL = 1 };
enum MvFf { MV_FF_NONE = 0, MV_FF_DENSE = 1, MV_FF_MOE = 2 };

struct MvLayer {
    asd_mavipel_layer_config c;
    std::unordered_map<std::string, const void*> t;   // weights by engine tensor name
    float* freq = nullptr;     // owned, [rot_dims / 2]
    int n_in = 0, ld_in = 0;   // rows of the stacked input projection; floats between its result's rows
    int mix_w = 0;             // columns of the stacked output projection
    int cache_row = 0;         // cached elements per position (0: none)
    int conv_ch = 0, conv_ring = 0;
    size_t conv_elems = 0;     // carried convolution inputs per sequence
    size_t state_elems = 0;    // recurrent state per (sequence, ring entry)
    const void* w(const char* name) const {
        auto it = t.find(name);
        return it == t.end() ? nullptr : it->second;
    }
    const float* f(const char* name) const { return static_cast<const float*>(w(name)); }
};

struct MvRun {
    int layer, pass;           // pass -1: outside the repeated span
    bool enters;               // first layer of a pass
    size_t cache_off = 0;      // elements from the pool start
    size_t conv_off = 0;       // floats from the state start
    size_t state_off = 0;
};

struct MvEngine : asd_mavipel_engine {
    asd_mavipel_config c;
    std::vector<MvLayer> layers;
    std::vector<MvRun> runs;
    std::unordered_map<std::string, const void*> g;   // global weights
    int f32 = 0, esz = 2;
    char* pool = nullptr;
    const int* page_table = nullptr;
    int num_pages = 0, max_seqs = 0, max_pages = 0;
    float* state = nullptr;
    // owned activations
    float *x = nullptr, *y = nullptr, *proj = nullptr, *conv = nullptr, *decay = nullptr, *gatev = nullptr, *rv = nullptr,
          *sc = nullptr, *orec = nullptr, *up = nullptr, *eout = nullptr, *rlog = nullptr, *rgate = nullptr;
    void *hn = nullptr, *mixed = nullptr, *act = nullptr, *xsel = nullptr;
    int *expert_of = nullptr, *counters = nullptr, *group_off = nullptr, *sorted_tok = nullptr, *slot_of = nullptr;
    std::vector<void*> owned;
    DenseRunner dn;
    EventProfiler prof;
    AttnSplit attn_ws;           // partial sums of the window attention's key shares (steps of few tokens)
    int* dev_error = nullptr;
    int device = 0;
    const void* gw(const char* name) const {
        auto it = g.find(name);
        return it == g.end() ? nullptr : it->second;
    }
};

template <typename T>
static int dev_alloc(MvEngine* e, T** p, size_t n) {
    void* q = nullptr;
    ASD_CUDA(cudaMalloc(&q, (n ? n : 1) * sizeof(T)));
    e->owned.push_back(q);
    *p = (T*)q;
    return 0;
}

enum MvProf { MV_DENSE = 0, MV_ATTN, MV_RECUR, MV_EXPERTS, MV_ROUTER, MV_ACT, MV_GLUE, MV_HEAD, MV_NCLASS };
#define MV_PROF(cls) ProfRegion _region(e->prof, cls, s)

static int linear(MvEngine* e, const SimtLinear& L, cudaStream_t s) {
    if (!e->f32 && e->dn.tc_linear && tc_linear_supports(L)) return launch_tc_linear(L, e->dev_error, s);
    return launch_simt_linear(L, s);
}

struct Batch {
    SeqIndex ix;
    const int* cu_q;
    const int* seq_slot;
    int nseq, max_qlen, max_kv_len;
};

// one delta-rule mixer over prepared inputs: vectors, recurrence, per-head norm and gate into `mixed` columns [col, ...)
static int delta_core(MvEngine* e, const Batch& b, const DeltaPrep& dp, const float* v, long long ldv, int dv, float* st,
                      const HeadNormGate& ng, int mix_w, int col, cudaStream_t s) {
    const int M = b.ix.M;
    {
        MV_PROF(MV_GLUE);
        if (launch_delta_prep(dp, M, s)) return -1;
    }
    {
        MV_PROF(MV_RECUR);
        if (launch_delta_recurrence(b.ix, b.cu_q, b.seq_slot, b.nseq, e->rv, e->sc, dp.general, v, ldv, dp.heads, dp.dk, dv,
                                    st, e->c.ring, e->orec, s))
            return -1;
    }
    MV_PROF(MV_GLUE);
    return launch_head_norm_gate(e->orec, ng, (char*)e->mixed + (size_t)col * e->esz, e->f32, mix_w, M, dp.heads, dv, s);
}

// mixer input hn [M][D] (engine type) -> mixed [M][mix_w] (engine type), the input of the stacked output projection
static int mix_channel_delta(MvEngine* e, const MvLayer& ly, const MvRun& run, int li, const Batch& b, cudaStream_t s) {
    const asd_mavipel_layer_config& c = ly.c;
    const int M = b.ix.M, D = e->c.width;
    const int nk = c.kv_heads * c.dim, nv = c.heads * c.vdim;
    {   // q | k | v | beta | decay-in | gate-in in one projection
        MV_PROF(MV_DENSE);
        if (e->dn.run(e->hn, ly.w("w_in"), e->proj, M, ly.n_in, D, ly.ld_in, li * 16 + 0, s)) return -1;
    }
    float* ring = e->state + run.conv_off;
    {
        MV_PROF(MV_GLUE);
        if (launch_short_conv(b.ix, e->proj, ly.ld_in, ly.f("conv_w"), c.conv, ly.conv_ch, ring, ly.conv_ring, e->conv, s))
            return -1;
        if (ly.conv_ring > 0 && launch_conv_commit(b.ix, b.cu_q, b.nseq, e->proj, ly.ld_in, ly.conv_ch, ring, ly.conv_ring, s))
            return -1;
        LowRankChannels dc;
        dc.w2 = ly.f("w_decay"), dc.bias = ly.f("b_decay"), dc.low = c.decay_rank, dc.n = c.heads * c.dim;
        dc.post = LRC_EXP_SOFTPLUS, dc.head_log_rate = ly.f("a_log"), dc.per_head = c.dim;
        if (launch_lowrank_channels(e->proj + 2 * nk + nv + c.heads, ly.ld_in, dc, e->decay, M, s)) return -1;
        LowRankChannels gc;
        gc.w2 = ly.f("w_gate"), gc.low = c.gate_rank, gc.n = nv, gc.post = LRC_SIGMOID;
        if (launch_lowrank_channels(e->proj + 2 * nk + nv + c.heads + c.decay_rank, ly.ld_in, gc, e->gatev, M, s)) return -1;
    }
    DeltaPrep dp;
    dp.q = e->conv, dp.k = e->conv + nk, dp.ld = ly.conv_ch, dp.decay = e->decay;
    dp.rv = e->rv, dp.sc = e->sc, dp.heads = c.heads, dp.kv_heads = c.kv_heads, dp.dk = c.dim, dp.general = 0;
    dp.q_scale = 1.f / sqrtf((float)c.dim);
    dp.beta = e->proj + 2 * nk + nv, dp.ld_beta = ly.ld_in;   // the raw betas stay in the projection's rows
    HeadNormGate ng;
    ng.gate = e->gatev, ng.ldg = nv, ng.w = ly.f("out_norm"), ng.w_per_head = 0, ng.gate_sigmoid = 0, ng.eps = e->c.eps;
    return delta_core(e, b, dp, e->conv + 2 * nk, ly.conv_ch, c.vdim, e->state + run.state_off, ng, ly.mix_w, 0, s);
}

static int mix_parallel(MvEngine* e, const MvLayer& ly, const MvRun& run, int li, const Batch& b, cudaStream_t s) {
    const asd_mavipel_layer_config& c = ly.c;
    const int M = b.ix.M, D = e->c.width, f32 = e->f32;
    const int nl = c.a_heads * c.a_dim + c.a_kv_heads * (c.a_dim + c.a_vdim), nr = c.r_heads * c.r_dim;
    {   // left q | k | v, right r | k | v | gate | rate | decay-in in one projection
        MV_PROF(MV_DENSE);
        if (e->dn.run(e->hn, ly.w("w_in"), e->proj, M, ly.n_in, D, ly.ld_in, li * 16 + 0, s)) return -1;
    }
    const TalkDims td{c.a_heads, c.a_kv_heads, c.a_dim, c.a_vdim, c.rot_dims, c.window, c.scale, c.softcap};
    const PagedRows cache{e->pool + run.cache_off * e->esz, f32, e->page_table, e->max_pages, e->c.page_size};
    {
        MV_PROF(MV_GLUE);
        if (launch_talk_post(b.ix, e->proj, ly.ld_in, td, ly.f("in_bias"), ly.f("q_norm"), ly.f("k_norm"), e->c.eps, ly.freq,
                             cache, s))
            return -1;
    }
    {
        MV_PROF(MV_ATTN);
        if (launch_talk_attention(b.ix, b.cu_q, b.seq_slot, b.nseq, b.max_qlen, b.max_kv_len, e->proj, ly.ld_in, td,
                                  ly.f("talk"), ly.f("sink"), cache, e->mixed, f32, ly.mix_w, c.left_scale, e->attn_ws, s))
            return -1;
    }
    float* r = e->proj + nl;
    {
        MV_PROF(MV_GLUE);
        LowRankChannels dc;
        dc.w2 = ly.f("w_decay"), dc.bias = ly.f("b_decay"), dc.low = c.r_decay_rank, dc.n = nr, dc.inner_tanh = 1;
        dc.post = LRC_EXP_SIGMOID, dc.rate = expf(-0.5f);
        if (launch_lowrank_channels(r + 5 * nr, ly.ld_in, dc, e->decay, M, s)) return -1;
    }
    DeltaPrep dp;
    dp.q = r, dp.k = r + nr, dp.ld = ly.ld_in, dp.decay = e->decay, dp.rate = r + 4 * nr, dp.rate_bias = ly.f("rate_bias");
    dp.rv = e->rv, dp.sc = e->sc, dp.heads = c.r_heads, dp.kv_heads = c.r_heads, dp.dk = c.r_dim, dp.general = 1;
    HeadNormGate ng;
    ng.gate = r + 3 * nr, ng.ldg = ly.ld_in, ng.w = ly.f("out_norm"), ng.w_per_head = 1, ng.gate_sigmoid = 1;
    ng.eps = e->c.eps, ng.scale = c.right_scale;
    return delta_core(e, b, dp, r + 2 * nr, ly.ld_in, c.r_dim, e->state + run.state_off, ng, ly.mix_w,
                      c.a_heads * c.a_vdim, s);
}

// hn = norm2(x) (engine type) -> x += ff(hn); the close also prepares what the next execution reads
static int feed_forward(MvEngine* e, const MvLayer& ly, int li, const Batch& b, RowClose& C, cudaStream_t s) {
    const asd_mavipel_layer_config& c = ly.c;
    const int M = b.ix.M, D = e->c.width, f32 = e->f32;
    if (c.ff_kind == MV_FF_DENSE) {
        {
            MV_PROF(MV_DENSE);
            if (e->dn.run(e->hn, ly.w("w_up"), e->up, M, c.ff, D, c.ff, li * 16 + 3, s)) return -1;
        }
        {
            MV_PROF(MV_ACT);
            if (launch_ff_act(e->up, e->act, f32, M, c.ff, 0, s)) return -1;
        }
        MV_PROF(MV_DENSE);
        if (e->dn.run(e->act, ly.w("w_down"), e->y, M, D, c.ff, D, li * 16 + 4, s)) return -1;
        C.y = e->y;
        return 0;
    }
    {   // router logits in fp32 on the CUDA cores in both modes, fused with the choice; gates = softmax over the chosen
        MV_PROF(MV_ROUTER);
        MoeRouterInput in{e->hn, f32, ly.w("router"), 1, D, e->rlog};
        in.bias = ly.f("router_b"), in.renorm = 1;
        if (launch_moe_route(nullptr, &in, M, c.experts, c.top, e->expert_of, e->rgate, e->counters, e->group_off,
                             e->sorted_tok, e->slot_of, s))
            return -1;
    }
    {
        MV_PROF(MV_EXPERTS);
        SimtLinear U;   // gate | up of every chosen (token, expert) pair
        U.a = e->hn, U.a_f32 = f32, U.lda = D;
        U.w = ly.w("w_gu"), U.w_f32 = f32, U.ldw = D, U.w_zs = (long long)2 * c.expert_ff * D;
        U.c = e->up, U.c_f32 = 1, U.ldc = 2 * c.expert_ff;
        U.M = M, U.N = 2 * c.expert_ff, U.K = D, U.Z = c.experts;
        U.group_off = e->group_off, U.gather = e->sorted_tok;
        if (linear(e, U, s)) return -1;
    }
    {
        MV_PROF(MV_ACT);
        if (launch_ff_act(e->up, e->act, f32, (long long)M * c.top, c.expert_ff, 1, s)) return -1;
    }
    {
        MV_PROF(MV_EXPERTS);
        SimtLinear W;
        W.a = e->act, W.a_f32 = f32, W.lda = c.expert_ff;
        W.w = ly.w("w_edown"), W.w_f32 = f32, W.ldw = c.expert_ff, W.w_zs = (long long)D * c.expert_ff;
        W.c = e->eout, W.c_f32 = 1, W.ldc = D;
        W.M = M, W.N = D, W.K = c.expert_ff, W.Z = c.experts;
        W.group_off = e->group_off;
        if (linear(e, W, s)) return -1;
    }
    C.expert_out = e->eout, C.slot_of = e->slot_of, C.gate = e->rgate, C.top = c.top;
    if (c.shared_ff > 0) {
        {
            MV_PROF(MV_DENSE);
            if (e->dn.run(e->hn, ly.w("w_sgu"), e->up, M, 2 * c.shared_ff, D, 2 * c.shared_ff, li * 16 + 5, s)) return -1;
        }
        {
            MV_PROF(MV_ACT);
            if (launch_ff_act(e->up, e->act, f32, M, c.shared_ff, 1, s)) return -1;
        }
        MV_PROF(MV_DENSE);
        if (e->dn.run(e->act, ly.w("w_sdown"), e->y, M, D, c.shared_ff, D, li * 16 + 6, s)) return -1;
        C.y = e->y;
    }
    return 0;
}

static int forward(MvEngine* e, const Batch& b, const int* logit_rows, int n_rows, float* logits, long long ld,
                   float* layer_out, cudaStream_t s) {
    const int D = e->c.width, M = b.ix.M, f32 = e->f32;
    const float eps = e->c.eps;
    const int nruns = (int)e->runs.size();
    auto base_close = [&]() {
        RowClose C;
        C.x_in = e->x, C.x_out = e->x, C.eps = eps, C.M = M, C.D = D, C.plain_w = 1, C.groups = e->c.norm_groups;
        return C;
    };
    // hn holds what the next execution's first projection reads, unless that execution enters a pass: then its own
    // close adds the pass's vector first
    auto open_next = [&](int r, RowClose& C) {
        if (r >= nruns || e->runs[r].enters) return;
        C.next_w = e->layers[e->runs[r].layer].f("norm1");
        C.hn = e->hn, C.hn_f32 = f32;
    };
    {
        MV_PROF(MV_GLUE);
        if (launch_embed_normed(b.ix, e->gw("embed"), f32, static_cast<const float*>(e->gw("embed_norm")), e->c.norm_groups,
                                eps, e->x, D, s))
            return -1;
        if (nruns && !e->runs[0].enters) {
            RowClose C = base_close();
            C.x_out = nullptr;
            open_next(0, C);
            if (launch_row_close(C, s)) return -1;
        }
    }
    for (int r = 0; r < nruns; ++r) {
        const MvRun& run = e->runs[r];
        const MvLayer& ly = e->layers[run.layer];
        const int li = run.layer;
        if (run.enters) {   // x <- x + step[pass], then this layer's first norm
            MV_PROF(MV_GLUE);
            RowClose C = base_close();
            C.bias = static_cast<const float*>(e->gw("loop_step")) + (size_t)run.pass * D;
            C.next_w = ly.f("norm1"), C.hn = e->hn, C.hn_f32 = f32;
            if (launch_row_close(C, s)) return -1;
        }
        if ((ly.c.type == MV_CHANNEL_DELTA ? mix_channel_delta(e, ly, run, li, b, s) : mix_parallel(e, ly, run, li, b, s)))
            return -1;
        {
            MV_PROF(MV_DENSE);
            if (e->dn.run(e->mixed, ly.w("w_o"), e->y, M, D, ly.mix_w, D, li * 16 + 2, s)) return -1;
        }
        {   // x += y; then the feed-forward's norm, or what the next execution reads
            MV_PROF(MV_GLUE);
            RowClose C = base_close();
            C.y = e->y;
            if (ly.c.ff_kind != MV_FF_NONE)
                C.next_w = ly.f("norm2"), C.hn = e->hn, C.hn_f32 = f32;
            else
                open_next(r + 1, C);
            if (launch_row_close(C, s)) return -1;
        }
        if (ly.c.ff_kind != MV_FF_NONE) {
            RowClose C = base_close();
            if (feed_forward(e, ly, li, b, C, s)) return -1;
            MV_PROF(MV_GLUE);
            open_next(r + 1, C);
            if (launch_row_close(C, s)) return -1;
        }
        if (layer_out)
            ASD_CUDA(cudaMemcpyAsync(layer_out + (size_t)r * M * D, e->x, sizeof(float) * M * D, cudaMemcpyDeviceToDevice, s));
    }
    if (n_rows > 0) {
        MV_PROF(MV_HEAD);
        RowClose C = base_close();
        C.x_out = nullptr, C.rows = logit_rows, C.next_w = static_cast<const float*>(e->gw("final_norm"));
        C.hn = e->xsel, C.hn_f32 = f32, C.M = n_rows;
        if (launch_row_close(C, s)) return -1;
        const int V = e->c.vocab;
        if (e->dn.run(e->xsel, e->gw("head"), logits, n_rows, V, D, ld ? (int)ld : V, (int)e->layers.size() * 16 + 2, s))
            return -1;
    }
    return 0;
}

// elements one execution's rows take in the pool, rounded up so that every execution starts on a 16-byte boundary
static size_t pool_elems(const MvEngine* e, const MvRun& r, int num_pages) {
    const size_t n = (size_t)num_pages * e->c.page_size * e->layers[r.layer].cache_row;
    return (n + 7) & ~(size_t)7;
}

static const char* const kLayerNames[] = {"norm1",  "norm2",  "w_in",    "w_o",  "conv_w", "a_log",     "w_decay", "b_decay",
                                          "w_gate", "out_norm", "in_bias", "q_norm", "k_norm", "talk",  "sink",    "rate_bias",
                                          "w_up",   "w_down", "router",  "router_b", "w_gu", "w_edown", "w_sgu",   "w_sdown"};
static const char* const kGlobalNames[] = {"embed", "embed_norm", "final_norm", "head", "loop_step"};

static std::vector<const char*> required(const MvLayer& ly) {
    std::vector<const char*> n = {"norm1", "w_in", "w_o", "w_decay", "b_decay", "out_norm"};
    if (ly.c.type == MV_CHANNEL_DELTA)
        n.insert(n.end(), {"conv_w", "a_log", "w_gate"});
    else
        n.insert(n.end(), {"rate_bias"});
    if (ly.c.ff_kind != MV_FF_NONE) n.push_back("norm2");
    if (ly.c.ff_kind == MV_FF_DENSE) n.insert(n.end(), {"w_up", "w_down"});
    if (ly.c.ff_kind == MV_FF_MOE) {
        n.insert(n.end(), {"router", "w_gu", "w_edown"});
        if (ly.c.shared_ff > 0) n.insert(n.end(), {"w_sgu", "w_sdown"});
    }
    return n;
}

}  // namespace asd

using namespace asd;

extern "C" {

asd_mavipel_engine_t* asd_mavipel_create(const asd_mavipel_config* cfg, const asd_mavipel_layer_config* layers) {
    if (!cfg || (cfg->n_layers > 0 && !layers)) {
        set_error("asd_mavipel_create: NULL config");
        return nullptr;
    }
    if (cfg->width <= 0 || cfg->vocab <= 0 || cfg->n_layers < 0 || cfg->max_tokens <= 0 || cfg->page_size <= 0 ||
        cfg->ring <= 0 || cfg->norm_groups <= 0 || cfg->width % cfg->norm_groups || (cfg->dtype != 0 && cfg->dtype != 1) ||
        cfg->loop_times < 0 ||
        (cfg->loop_times > 0 && !(0 <= cfg->loop_start && cfg->loop_start < cfg->loop_stop && cfg->loop_stop <= cfg->n_layers))) {
        set_error("asd_mavipel_create: bad sizes");
        return nullptr;
    }
    MvEngine* e = new MvEngine();
    e->c = *cfg;
    e->f32 = e->dn.f32 = cfg->dtype;
    e->esz = cfg->dtype ? 4 : 2;
    cudaGetDevice(&e->device);
    const size_t MT = cfg->max_tokens, D = cfg->width;
    size_t ld_in = 4, conv = 1, nk = 1, nv = 1, rvn = 1, heads = 1, mixw = 1, upw = 1, actw = 1, E = 1, top = 1, share = 0;
    auto fail = [&](const char* what, int l) {
        set_error("asd_mavipel_create: %s (layer %d)", what, l);
        asd_mavipel_destroy(e);
        return nullptr;
    };
    for (int l = 0; l < cfg->n_layers; ++l) {
        MvLayer ly;
        ly.c = layers[l];
        const auto& c = ly.c;
        if (c.type == MV_CHANNEL_DELTA) {
            if (c.heads <= 0 || c.kv_heads <= 0 || c.heads % c.kv_heads || c.dim <= 0 || c.vdim <= 0 || c.conv <= 0 ||
                c.decay_rank <= 0 || c.gate_rank <= 0)
                return fail("bad gated delta rule sizes", l);
            ly.conv_ch = 2 * c.kv_heads * c.dim + c.heads * c.vdim;
            ly.n_in = ly.conv_ch + c.heads + c.decay_rank + c.gate_rank;
            ly.mix_w = c.heads * c.vdim;
            // inputs of the last conv - 1 positions, for each of the `ring` positions a forward may start after
            ly.conv_ring = c.conv > 1 ? c.conv - 1 + cfg->ring - 1 : 0;
            ly.conv_elems = (size_t)ly.conv_ring * ly.conv_ch;
            ly.state_elems = (size_t)c.heads * c.dim * c.vdim;
            conv = std::max(conv, (size_t)ly.conv_ch);
            nk = std::max(nk, (size_t)c.heads * c.dim);
            nv = std::max(nv, (size_t)c.heads * c.vdim);
            rvn = std::max(rvn, (size_t)c.heads * 4 * c.dim);
            heads = std::max(heads, (size_t)c.heads);
        } else if (c.type == MV_PARALLEL) {
            if (c.a_heads <= 0 || c.a_heads > 32 || c.a_kv_heads <= 0 || c.a_heads % c.a_kv_heads || c.a_dim <= 0 ||
                c.a_vdim <= 0 || c.a_vdim > 256 || c.rot_dims < 0 || c.rot_dims > c.a_dim || (c.rot_dims & 1) || c.window <= 0)
                return fail("bad window attention sizes", l);
            if (c.r_heads <= 0 || c.r_dim <= 0 || c.r_decay_rank <= 0) return fail("bad generalised delta rule sizes", l);
            const int nr = c.r_heads * c.r_dim;
            ly.n_in = c.a_heads * c.a_dim + c.a_kv_heads * (c.a_dim + c.a_vdim) + 5 * nr + c.r_decay_rank;
            ly.mix_w = c.a_heads * c.a_vdim + nr;
            ly.cache_row = c.a_kv_heads * (c.a_dim + c.a_vdim);
            share = std::max(share, (size_t)c.a_heads * (c.a_vdim + 2));
            ly.state_elems = (size_t)c.r_heads * c.r_dim * c.r_dim;
            nk = std::max(nk, (size_t)nr);
            nv = std::max(nv, (size_t)nr);
            rvn = std::max(rvn, (size_t)5 * nr);
            heads = std::max(heads, (size_t)c.r_heads);
            const int half = c.rot_dims / 2;
            std::vector<float> f(half > 0 ? half : 1, 0.f);
            for (int i = 0; i < half; ++i) f[i] = (float)pow((double)c.rot_base, -2.0 * i / (double)c.rot_dims);
            if (dev_alloc(e, &ly.freq, f.size()) ||
                cudaMemcpy(ly.freq, f.data(), f.size() * sizeof(float), cudaMemcpyHostToDevice) != cudaSuccess)
                return fail("device allocation failed", l);
        } else {
            return fail("unknown mixer type", l);
        }
        if (c.ff_kind == MV_FF_DENSE) {
            if (c.ff <= 0) return fail("bad feed-forward size", l);
            upw = std::max(upw, (size_t)c.ff);
            actw = std::max(actw, (size_t)c.ff);
        } else if (c.ff_kind == MV_FF_MOE) {
            if (c.experts <= 0 || c.top <= 0 || c.top > c.experts || c.expert_ff <= 0 || c.shared_ff < 0)
                return fail("bad expert sizes", l);
            upw = std::max(upw, std::max((size_t)c.top * 2 * c.expert_ff, (size_t)2 * c.shared_ff));
            actw = std::max(actw, std::max((size_t)c.top * c.expert_ff, (size_t)c.shared_ff));
            E = std::max(E, (size_t)c.experts);
            top = std::max(top, (size_t)c.top);
        } else if (c.ff_kind != MV_FF_NONE) {
            return fail("unknown feed-forward kind", l);
        }
        ly.ld_in = (ly.n_in + 3) & ~3;
        ld_in = std::max(ld_in, (size_t)ly.ld_in);
        mixw = std::max(mixw, (size_t)ly.mix_w);
        e->layers.push_back(ly);
    }
    auto add = [&](int l, int pass, bool enters) { e->runs.push_back(MvRun{l, pass, enters}); };
    if (cfg->loop_times == 0) {
        for (int l = 0; l < cfg->n_layers; ++l) add(l, -1, false);
    } else {
        for (int l = 0; l < cfg->loop_start; ++l) add(l, -1, false);
        for (int t = 0; t < cfg->loop_times; ++t)
            for (int l = cfg->loop_start; l < cfg->loop_stop; ++l) add(l, t, l == cfg->loop_start);
        for (int l = cfg->loop_stop; l < cfg->n_layers; ++l) add(l, -1, false);
    }
    int rc = 0;
    rc |= dev_alloc(e, &e->x, MT * D);
    rc |= dev_alloc(e, &e->y, MT * D);
    rc |= dev_alloc(e, &e->proj, MT * ld_in);
    rc |= dev_alloc(e, &e->conv, MT * conv);
    rc |= dev_alloc(e, &e->decay, MT * nk);
    rc |= dev_alloc(e, &e->gatev, MT * nv);
    rc |= dev_alloc(e, &e->rv, MT * rvn);
    rc |= dev_alloc(e, &e->sc, MT * heads * 4);
    rc |= dev_alloc(e, &e->orec, MT * nv);
    rc |= dev_alloc(e, &e->up, MT * upw);
    rc |= dev_alloc(e, &e->eout, MT * top * D);
    rc |= dev_alloc(e, &e->rlog, MT * E);
    rc |= dev_alloc(e, &e->rgate, MT * top);
    rc |= dev_alloc(e, (char**)&e->hn, MT * D * e->esz);
    rc |= dev_alloc(e, (char**)&e->mixed, MT * mixw * e->esz);
    rc |= dev_alloc(e, (char**)&e->act, MT * actw * e->esz);
    rc |= dev_alloc(e, (char**)&e->xsel, MT * D * e->esz);
    rc |= dev_alloc(e, &e->expert_of, MT * top);
    rc |= dev_alloc(e, &e->counters, 2 * E + 1);
    rc |= dev_alloc(e, &e->group_off, E + 1);
    rc |= dev_alloc(e, &e->sorted_tok, MT * top);
    rc |= dev_alloc(e, &e->slot_of, MT * top);
    // key shares are used while CTAs are fewer than half the SMs: at most 148 x 8 (token, share) pairs
    e->attn_ws.o_elems = (long long)(148 * 8 * share);
    if (share) {
        rc |= dev_alloc(e, &e->attn_ws.o, (size_t)e->attn_ws.o_elems);
        rc |= dev_alloc(e, &e->attn_ws.ml, MT);      // arrival counters of the key shares, one per token
        e->attn_ws.rows = (long long)MT;
        if (!rc && cudaMemset(e->attn_ws.ml, 0, MT * sizeof(float)) != cudaSuccess) rc = -1;
    }
    rc |= dev_alloc(e, &e->dev_error, 1);
    if (!rc && cudaMemset(e->dev_error, 0, sizeof(int)) != cudaSuccess) rc = -1;
    if (rc) {
        asd_mavipel_destroy(e);
        return nullptr;
    }
    return e;
}

void asd_mavipel_destroy(asd_mavipel_engine_t* h) {
    MvEngine* e = static_cast<MvEngine*>(h);
    if (!e) return;
    for (void* p : e->owned) cudaFree(p);
    delete e;
}

int asd_mavipel_set_tensor(asd_mavipel_engine_t* h, int layer, const char* name, const void* data) {
    MvEngine* e = static_cast<MvEngine*>(h);
    if (!e || !name || !data) return set_error("asd_mavipel_set_tensor: NULL argument");
    if (layer >= (int)e->layers.size() || layer < -1) return set_error("asd_mavipel_set_tensor: bad layer %d", layer);
    bool known = false;
    if (layer < 0) {
        for (const char* n : kGlobalNames) known |= !strcmp(n, name);
        if (known) e->g[name] = data;
    } else {
        for (const char* n : kLayerNames) known |= !strcmp(n, name);
        if (known) e->layers[layer].t[name] = data;
    }
    if (!known) return set_error("asd_mavipel_set_tensor: unknown tensor %s (layer %d)", name, layer);
    e->dn.clear();
    return 0;
}

size_t asd_mavipel_cache_bytes(const asd_mavipel_engine_t* h, int num_pages) {
    const MvEngine* e = static_cast<const MvEngine*>(h);
    if (!e) return 0;
    size_t n = 0;
    for (const MvRun& r : e->runs) n += pool_elems(e, r, num_pages);
    return n * e->esz;
}

size_t asd_mavipel_state_bytes(const asd_mavipel_engine_t* h, int max_seqs) {
    const MvEngine* e = static_cast<const MvEngine*>(h);
    if (!e) return 0;
    size_t n = 0;
    for (const MvRun& r : e->runs) {
        const MvLayer& ly = e->layers[r.layer];
        n += (size_t)max_seqs * (ly.conv_elems + (size_t)e->c.ring * ly.state_elems);
    }
    return n * sizeof(float);
}

int asd_mavipel_set_cache(asd_mavipel_engine_t* h, void* pool, int num_pages, const int32_t* page_table, int max_seqs,
                          int max_pages_per_seq, float* state) {
    MvEngine* e = static_cast<MvEngine*>(h);
    if (!e || !pool || !page_table || !state || num_pages <= 0 || max_seqs <= 0 || max_pages_per_seq <= 0)
        return set_error("asd_mavipel_set_cache: bad arguments");
    e->pool = static_cast<char*>(pool);
    e->num_pages = num_pages, e->page_table = page_table, e->max_seqs = max_seqs, e->max_pages = max_pages_per_seq;
    e->state = state;
    size_t off = 0, soff = 0;
    for (MvRun& r : e->runs) {
        const MvLayer& ly = e->layers[r.layer];
        r.cache_off = off;
        off += pool_elems(e, r, num_pages);
        r.conv_off = soff;
        soff += (size_t)max_seqs * ly.conv_elems;
        r.state_off = soff;
        soff += (size_t)max_seqs * e->c.ring * ly.state_elems;
    }
    return 0;
}

int asd_mavipel_set_option(asd_mavipel_engine_t* h, const char* name, int value) {
    MvEngine* e = static_cast<MvEngine*>(h);
    if (!e || !name) return set_error("asd_mavipel_set_option: NULL argument");
    if (!strcmp(name, "tc_linear")) {
        e->dn.tc_linear = value;
        return 0;
    }
    if (!strcmp(name, "tc_min_rows")) {
        e->dn.tc_min_rows = value > 0 ? value : 1 << 30;
        e->dn.clear();
        return 0;
    }
    if (!strcmp(name, "attn_mma")) {
        e->attn_ws.tiled = value;
        return 0;
    }
    if (!strcmp(name, "profile")) {
        e->prof.on = value;
        e->prof.reset();
        return 0;
    }
    return set_error("asd_mavipel_set_option: unknown option %s", name);
}

int asd_mavipel_forward(asd_mavipel_engine_t* h, const int32_t* tokens, const int32_t* positions,
                        const int32_t* token_slot, int M, const int32_t* cu_q, const int32_t* seq_slot, int nseq,
                        int max_qlen, int max_kv_len, const int32_t* logit_rows, int n_logit_rows, float* logits_out,
                        long long logits_ld, float* layer_out, void* stream) {
    MvEngine* e = static_cast<MvEngine*>(h);
    if (!e) return set_error("asd_mavipel_forward: NULL engine");
    if (M <= 0 || M > e->c.max_tokens) return set_error("asd_mavipel_forward: M = %d outside 1..%d", M, e->c.max_tokens);
    if (!e->pool) return set_error("asd_mavipel_forward: cache not set");
    for (const char* n : {"embed", "embed_norm", "final_norm", "head"})
        if (!e->gw(n)) return set_error("asd_mavipel_forward: tensor %s not set", n);
    if (e->c.loop_times > 0 && !e->gw("loop_step")) return set_error("asd_mavipel_forward: the repeated span's vectors are not set");
    for (size_t l = 0; l < e->layers.size(); ++l)
        for (const char* n : required(e->layers[l]))
            if (!e->layers[l].w(n)) return set_error("asd_mavipel_forward: layer %d has no tensor %s", (int)l, n);
    if (!tokens || !positions || !token_slot || !cu_q || !seq_slot || nseq <= 0 || max_qlen <= 0)
        return set_error("asd_mavipel_forward: bad index arguments");
    if (max_kv_len > e->max_pages * e->c.page_size)
        return set_error("asd_mavipel_forward: length bound %d exceeds the page table", max_kv_len);
    if (n_logit_rows > 0 && !logits_out) return set_error("asd_mavipel_forward: logits_out is NULL");
    if (n_logit_rows > e->c.max_tokens) return set_error("asd_mavipel_forward: too many logit rows");
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev != e->device) return set_error("asd_mavipel_forward: called on device %d, engine lives on %d", dev, e->device);
    const Batch b{SeqIndex{tokens, positions, token_slot, M}, cu_q, seq_slot, nseq, max_qlen, max_kv_len};
    return forward(e, b, logit_rows, logit_rows ? n_logit_rows : (n_logit_rows > 0 ? M : 0), logits_out, logits_ld,
                   layer_out, static_cast<cudaStream_t>(stream));
}

int asd_mavipel_profile_read(asd_mavipel_engine_t* h, float* ms_by_class, int* launches_by_class, int nclass) {
    MvEngine* e = static_cast<MvEngine*>(h);
    if (!e || !ms_by_class || nclass < MV_NCLASS) return set_error("asd_mavipel_profile_read: bad argument");
    ASD_CUDA(e->prof.read(ms_by_class, launches_by_class, nclass));
    return 0;
}

int asd_mavipel_device_error(asd_mavipel_engine_t* h) {
    MvEngine* e = static_cast<MvEngine*>(h);
    if (!e) return set_error("asd_mavipel_device_error: NULL engine");
    int v = 0;
    ASD_CUDA(cudaMemcpy(&v, e->dev_error, sizeof(int), cudaMemcpyDeviceToHost));
    if (v) return set_error("a Mavipel kernel gave up a bounded wait (tcgen05 linear)");
    return 0;
}

}  // extern "C"
