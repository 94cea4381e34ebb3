// Lukopel family forward engine: one opaque handle per model.  asd_lukopel_forward runs, on the caller's stream and with
// no host synchronisation,
//   scaled embedding + position vector, copied into S residual streams -> for every layer execution
//   [ read the streams, norm, attention mixer, write the streams; read, norm, feed-forward, write ] ->
//   sum of the streams, final norm of the wanted rows, head.
// A layer's mixer is grouped-query softmax attention in one of two forms that differ in parameters only: query/key norm
// per head or over the whole projection, biased or unbiased projections, a query factor that grows with the position
// and / or one per head, unit-RMS values, a learned bias per (distance bucket, head), a causal mask that may be cut
// into chunks, softmax weights mixed across the heads, a sigmoid gate per head.  The feed-forward is a biased two-matrix
// layer with a squared relu.  Layers of a repeated span execute several times with the same weights and a cache per
// execution.  Every step is a building block of blocks.h; dense bf16 projections go to the tcgen05 GEMMs when their
// shape fits (dense.h).  The streams, norms, scores and softmax weights are fp32 in both element types.
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

struct asd_lukopel_engine {};

namespace asd {

struct LkLayer {
    asd_lukopel_layer_config c;
    std::unordered_map<std::string, const void*> t;   // weights by engine tensor name
    int n_in = 0, ld_in = 0;   // rows of the stacked input projection; floats between its result's rows
    int mix_w = 0;             // columns of the output projection
    int cache_row = 0;         // cached elements per position
    const void* w(const char* name) const {
        auto it = t.find(name);
        return it == t.end() ? nullptr : it->second;
    }
    const float* f(const char* name) const { return static_cast<const float*>(w(name)); }
};

struct LkRun {
    int layer, pass;           // pass -1: outside the repeated span
    size_t cache_off = 0;      // elements from the pool start
};

struct LkEngine : asd_lukopel_engine {
    asd_lukopel_config c;
    std::vector<LkLayer> layers;
    std::vector<LkRun> runs;
    std::unordered_map<std::string, const void*> g;   // global weights
    int f32 = 0, esz = 2;
    char* pool = nullptr;
    const int* page_table = nullptr;
    int num_pages = 0, max_seqs = 0, max_pages = 0;
    // owned activations
    float *xs = nullptr, *y = nullptr, *proj = nullptr, *up = nullptr;
    void *hn = nullptr, *mixed = nullptr, *act = nullptr, *xsel = nullptr;
    MixWork attn_ws;
    std::vector<void*> owned;
    DenseRunner dn;
    EventProfiler prof;
    int* dev_error = nullptr;
    int device = 0;
    const void* gw(const char* name) const {
        auto it = g.find(name);
        return it == g.end() ? nullptr : it->second;
    }
};

template <typename T>
static int dev_alloc(LkEngine* e, T** p, size_t n) {
    void* q = nullptr;
    ASD_CUDA(cudaMalloc(&q, (n ? n : 1) * sizeof(T)));
    e->owned.push_back(q);
    *p = (T*)q;
    return 0;
}

enum LkProf { LK_DENSE = 0, LK_ATTN, LK_ACT, LK_GLUE, LK_HEAD, LK_NCLASS };
#define LK_PROF(cls) ProfRegion _region(e->prof, cls, s)

struct LkBatch {
    SeqIndex ix;
    const int* cu_q;
    const int* seq_slot;
    int nseq, max_qlen, max_kv_len;
};

static MixDims mix_dims(const asd_lukopel_layer_config& c) {
    return MixDims{c.heads, c.kv_heads, c.dim, c.vdim, c.chunk, c.scale};
}

// mixer input hn [M][D] (engine type) -> mixed [M][heads * vdim] (engine type), the input of the output projection
static int mixer(LkEngine* e, const LkLayer& ly, const LkRun& run, int li, const LkBatch& b, cudaStream_t s) {
    const asd_lukopel_layer_config& c = ly.c;
    const int M = b.ix.M, D = e->c.width;
    {   // q | k | v (| one gate value per head) in one projection
        LK_PROF(LK_DENSE);
        if (e->dn.run(e->hn, ly.w("w_in"), e->proj, M, ly.n_in, D, ly.ld_in, li * 16 + 0, s)) return -1;
    }
    const MixDims md = mix_dims(c);
    const PagedRows cache{e->pool + run.cache_off * e->esz, e->f32, e->page_table, e->max_pages, e->c.page_size};
    {
        LK_PROF(LK_GLUE);
        MixPost p;
        p.bias = ly.f("in_bias"), p.q_norm = ly.f("q_norm"), p.k_norm = ly.f("k_norm"), p.norm_whole = c.norm_whole;
        p.temp_coef = c.temp_coef, p.temp_every = c.temp_every, p.head_factor = ly.f("head_factor");
        p.v_unit = c.v_unit, p.eps = e->c.eps;
        if (launch_mix_post(b.ix, e->proj, ly.ld_in, md, p, cache, s)) return -1;
    }
    LK_PROF(LK_ATTN);
    const float* gate = c.gated ? e->proj + c.heads * c.dim + c.kv_heads * (c.dim + c.vdim) : nullptr;
    return launch_mix_attention(b.ix, b.cu_q, b.seq_slot, b.nseq, b.max_qlen, b.max_kv_len, e->proj, ly.ld_in, md,
                                ly.f("dist_bias"), c.far, ly.f("talk"), gate, ly.ld_in, cache, e->mixed, e->f32, ly.mix_w,
                                e->attn_ws, s);
}

static int forward(LkEngine* e, const LkBatch& b, const int* logit_rows, int n_rows, float* logits, long long ld,
                   float* layer_out, cudaStream_t s) {
    const int D = e->c.width, M = b.ix.M, f32 = e->f32, S = e->c.streams;
    const int nruns = (int)e->runs.size();
    auto base_close = [&]() {
        StreamClose C;
        C.xs = e->xs, C.eps = e->c.eps, C.M = M, C.S = S, C.D = D;
        return C;
    };
    // what a sublayer reads: the streams' weighted sum (plain sum where a layer has no read weights), normed
    auto open_sub = [&](StreamClose& C, const LkLayer& ly, int sub) {
        C.read = ly.f(sub == 1 ? "hc1_read" : "hc2_read");
        C.want_sum = C.read ? 0 : 1;
        C.next_w = ly.f(sub == 1 ? "norm1" : "norm2");
        C.hn = e->hn, C.hn_f32 = f32;
    };
    auto open_next = [&](StreamClose& C, int r) {
        if (r < nruns) open_sub(C, e->layers[e->runs[r].layer], 1);
    };
    {
        LK_PROF(LK_GLUE);
        if (launch_embed_streams(b.ix, e->gw("embed"), e->gw("pos"), f32, e->c.embed_scale, e->xs, S, D, s)) return -1;
        if (nruns) {
            StreamClose C = base_close();
            open_next(C, 0);
            if (launch_stream_close(C, s)) return -1;
        }
    }
    for (int r = 0; r < nruns; ++r) {
        const LkRun& run = e->runs[r];
        const LkLayer& ly = e->layers[run.layer];
        const int li = run.layer;
        if (mixer(e, ly, run, li, b, s)) return -1;
        {
            LK_PROF(LK_DENSE);
            if (e->dn.run(e->mixed, ly.w("w_o"), e->y, M, D, ly.mix_w, D, li * 16 + 2, s)) return -1;
        }
        {   // the streams take the mixer's result; then the feed-forward's input, or the next execution's
            LK_PROF(LK_GLUE);
            StreamClose C = base_close();
            C.y = e->y, C.y_bias = ly.f("o_bias"), C.mix = ly.f("hc1_mix"), C.write = ly.f("hc1_write");
            if (ly.c.ff_kind)
                open_sub(C, ly, 2);
            else
                open_next(C, r + 1);
            if (launch_stream_close(C, s)) return -1;
        }
        if (ly.c.ff_kind) {
            {
                LK_PROF(LK_DENSE);
                if (e->dn.run(e->hn, ly.w("w_up"), e->up, M, ly.c.ff, D, ly.c.ff, li * 16 + 3, s)) return -1;
            }
            {
                LK_PROF(LK_ACT);
                if (launch_ff_act(e->up, e->act, f32, M, ly.c.ff, 2, s, ly.f("up_bias"))) return -1;
            }
            {
                LK_PROF(LK_DENSE);
                if (e->dn.run(e->act, ly.w("w_down"), e->y, M, D, ly.c.ff, D, li * 16 + 4, s)) return -1;
            }
            LK_PROF(LK_GLUE);
            StreamClose C = base_close();
            C.y = e->y, C.y_bias = ly.f("down_bias"), C.mix = ly.f("hc2_mix"), C.write = ly.f("hc2_write");
            open_next(C, r + 1);
            if (launch_stream_close(C, s)) return -1;
        }
        if (layer_out) {
            StreamClose C = base_close();
            C.want_sum = 1, C.u_out = layer_out + (size_t)r * M * D;
            if (launch_stream_close(C, s)) return -1;
        }
    }
    if (n_rows > 0) {
        LK_PROF(LK_HEAD);
        StreamClose C = base_close();
        C.rows = logit_rows, C.want_sum = 1, C.next_w = static_cast<const float*>(e->gw("final_norm"));
        C.hn = e->xsel, C.hn_f32 = f32, C.M = n_rows;
        if (launch_stream_close(C, s)) return -1;
        const int V = e->c.vocab;
        if (e->dn.run(e->xsel, e->gw("head"), logits, n_rows, V, D, ld ? (int)ld : V, (int)e->layers.size() * 16 + 2, s))
            return -1;
    }
    return 0;
}

// elements one execution's rows take in the pool, rounded up so that every execution starts on a 16-byte boundary
static size_t pool_elems(const LkEngine* e, const LkRun& r, int num_pages) {
    const size_t n = (size_t)num_pages * e->c.page_size * e->layers[r.layer].cache_row;
    return (n + 7) & ~(size_t)7;
}

static const char* const kLayerNames[] = {"norm1",   "norm2",     "w_in",      "w_o",     "in_bias",  "o_bias",   "q_norm",
                                          "k_norm",  "dist_bias", "talk",      "head_factor", "w_up", "up_bias",  "w_down",
                                          "down_bias", "hc1_read", "hc1_write", "hc1_mix", "hc2_read", "hc2_write", "hc2_mix"};
static const char* const kGlobalNames[] = {"embed", "pos", "final_norm", "head"};

}  // namespace asd

using namespace asd;

extern "C" {

asd_lukopel_engine_t* asd_lukopel_create(const asd_lukopel_config* cfg, const asd_lukopel_layer_config* layers) {
    if (!cfg || (cfg->n_layers > 0 && !layers)) {
        set_error("asd_lukopel_create: NULL config");
        return nullptr;
    }
    if (cfg->width <= 0 || cfg->vocab <= 0 || cfg->n_layers < 0 || cfg->max_tokens <= 0 || cfg->page_size <= 0 ||
        cfg->streams <= 0 || cfg->streams > 16 || (cfg->dtype != 0 && cfg->dtype != 1) || cfg->loop_times < 0 ||
        (cfg->loop_times > 0 && !(0 <= cfg->loop_start && cfg->loop_start < cfg->loop_stop && cfg->loop_stop <= cfg->n_layers))) {
        set_error("asd_lukopel_create: bad sizes");
        return nullptr;
    }
    LkEngine* e = new LkEngine();
    e->c = *cfg;
    e->f32 = e->dn.f32 = cfg->dtype;
    e->esz = cfg->dtype ? 4 : 2;
    cudaGetDevice(&e->device);
    const size_t MT = cfg->max_tokens, D = cfg->width;
    size_t ld_in = 4, mixw = 1, upw = 1, heads = 1;
    auto fail = [&](const char* what, int l) {
        set_error("asd_lukopel_create: %s (layer %d)", what, l);
        asd_lukopel_destroy(e);
        return nullptr;
    };
    for (int l = 0; l < cfg->n_layers; ++l) {
        LkLayer ly;
        ly.c = layers[l];
        const auto& c = ly.c;
        if (mix_attention_check(mix_dims(c), 0)) {
            asd_lukopel_destroy(e);
            return nullptr;
        }
        if (c.far < 0 || c.temp_every < 0) return fail("bad attention constants", l);
        if (c.ff_kind != 0 && c.ff_kind != 1) return fail("unknown feed-forward kind", l);
        if (c.ff_kind == 1 && c.ff <= 0) return fail("bad feed-forward size", l);
        ly.n_in = c.heads * c.dim + c.kv_heads * (c.dim + c.vdim) + (c.gated ? c.heads : 0);
        ly.ld_in = (ly.n_in + 3) & ~3;
        ly.mix_w = c.heads * c.vdim;
        ly.cache_row = c.kv_heads * (c.dim + c.vdim);
        ld_in = std::max(ld_in, (size_t)ly.ld_in);
        mixw = std::max(mixw, (size_t)ly.mix_w);
        heads = std::max(heads, (size_t)c.heads);
        if (c.ff_kind) upw = std::max(upw, (size_t)c.ff);
        e->layers.push_back(ly);
    }
    auto add = [&](int l, int pass) { e->runs.push_back(LkRun{l, pass}); };
    if (cfg->loop_times == 0) {
        for (int l = 0; l < cfg->n_layers; ++l) add(l, -1);
    } else {
        for (int l = 0; l < cfg->loop_start; ++l) add(l, -1);
        for (int t = 0; t < cfg->loop_times; ++t)
            for (int l = cfg->loop_start; l < cfg->loop_stop; ++l) add(l, t);
        for (int l = cfg->loop_stop; l < cfg->n_layers; ++l) add(l, -1);
    }
    int rc = 0;
    rc |= dev_alloc(e, &e->xs, MT * cfg->streams * D);
    rc |= dev_alloc(e, &e->y, MT * D);
    rc |= dev_alloc(e, &e->proj, MT * ld_in);
    rc |= dev_alloc(e, &e->up, MT * upw);
    rc |= dev_alloc(e, (char**)&e->hn, MT * D * e->esz);
    rc |= dev_alloc(e, (char**)&e->mixed, MT * mixw * e->esz);
    rc |= dev_alloc(e, (char**)&e->act, MT * upw * e->esz);
    rc |= dev_alloc(e, (char**)&e->xsel, MT * D * e->esz);
    // statistics of up to 32 key shares for steps of few tokens (one share otherwise); partial results of 2048
    // (token, share) pairs
    e->attn_ws.stats_elems = (long long)(2 * std::max<size_t>(MT, 32 * 64) * heads);
    e->attn_ws.part_elems = (long long)(2048 * mixw);
    rc |= dev_alloc(e, &e->attn_ws.stats, (size_t)e->attn_ws.stats_elems);
    rc |= dev_alloc(e, &e->attn_ws.part, (size_t)e->attn_ws.part_elems);
    e->attn_ws.score_elems = 8ll << 20;      // scores of steps of few tokens: tokens x heads x keys
    rc |= dev_alloc(e, &e->attn_ws.scores, (size_t)e->attn_ws.score_elems);
    rc |= dev_alloc(e, &e->dev_error, 1);
    if (!rc && cudaMemset(e->dev_error, 0, sizeof(int)) != cudaSuccess) rc = -1;
    if (rc) {
        asd_lukopel_destroy(e);
        return nullptr;
    }
    return e;
}

void asd_lukopel_destroy(asd_lukopel_engine_t* h) {
    LkEngine* e = static_cast<LkEngine*>(h);
    if (!e) return;
    for (void* p : e->owned) cudaFree(p);
    delete e;
}

int asd_lukopel_set_tensor(asd_lukopel_engine_t* h, int layer, const char* name, const void* data) {
    LkEngine* e = static_cast<LkEngine*>(h);
    if (!e || !name || !data) return set_error("asd_lukopel_set_tensor: NULL argument");
    if (layer >= (int)e->layers.size() || layer < -1) return set_error("asd_lukopel_set_tensor: bad layer %d", layer);
    bool known = false;
    if (layer < 0) {
        for (const char* n : kGlobalNames) known |= !strcmp(n, name);
        if (known) e->g[name] = data;
    } else {
        for (const char* n : kLayerNames) known |= !strcmp(n, name);
        if (known) e->layers[layer].t[name] = data;
    }
    if (!known) return set_error("asd_lukopel_set_tensor: unknown tensor %s (layer %d)", name, layer);
    e->dn.clear();
    return 0;
}

size_t asd_lukopel_cache_bytes(const asd_lukopel_engine_t* h, int num_pages) {
    const LkEngine* e = static_cast<const LkEngine*>(h);
    if (!e) return 0;
    size_t n = 0;
    for (const LkRun& r : e->runs) n += pool_elems(e, r, num_pages);
    return n * e->esz;
}

size_t asd_lukopel_state_bytes(const asd_lukopel_engine_t*, int) { return 0; }   // nothing is carried besides the cache

int asd_lukopel_set_cache(asd_lukopel_engine_t* h, void* pool, int num_pages, const int32_t* page_table, int max_seqs,
                          int max_pages_per_seq, float* /*state*/) {
    LkEngine* e = static_cast<LkEngine*>(h);
    if (!e || !pool || !page_table || num_pages <= 0 || max_seqs <= 0 || max_pages_per_seq <= 0)
        return set_error("asd_lukopel_set_cache: bad arguments");
    e->pool = static_cast<char*>(pool);
    e->num_pages = num_pages, e->page_table = page_table, e->max_seqs = max_seqs, e->max_pages = max_pages_per_seq;
    size_t off = 0;
    for (LkRun& r : e->runs) {
        r.cache_off = off;
        off += pool_elems(e, r, num_pages);
    }
    return 0;
}

int asd_lukopel_set_option(asd_lukopel_engine_t* h, const char* name, int value) {
    LkEngine* e = static_cast<LkEngine*>(h);
    if (!e || !name) return set_error("asd_lukopel_set_option: NULL argument");
    if (!strcmp(name, "tc_linear")) {
        e->dn.tc_linear = value;
        return 0;
    }
    if (!strcmp(name, "tc_min_rows")) {
        e->dn.tc_min_rows = value > 0 ? value : 1 << 30;
        e->dn.clear();
        return 0;
    }
    if (!strcmp(name, "attn_general")) {
        e->attn_ws.mode = value ? 1 : 0;
        return 0;
    }
    if (!strcmp(name, "profile")) {
        e->prof.on = value;
        e->prof.reset();
        return 0;
    }
    return set_error("asd_lukopel_set_option: unknown option %s", name);
}

int asd_lukopel_forward(asd_lukopel_engine_t* h, const int32_t* tokens, const int32_t* positions,
                        const int32_t* token_slot, int M, const int32_t* cu_q, const int32_t* seq_slot, int nseq,
                        int max_qlen, int max_kv_len, const int32_t* logit_rows, int n_logit_rows, float* logits_out,
                        long long logits_ld, float* layer_out, void* stream) {
    LkEngine* e = static_cast<LkEngine*>(h);
    if (!e) return set_error("asd_lukopel_forward: NULL engine");
    if (M <= 0 || M > e->c.max_tokens) return set_error("asd_lukopel_forward: M = %d outside 1..%d", M, e->c.max_tokens);
    if (!e->pool) return set_error("asd_lukopel_forward: cache not set");
    for (const char* n : {"embed", "final_norm", "head"})
        if (!e->gw(n)) return set_error("asd_lukopel_forward: tensor %s not set", n);
    for (size_t l = 0; l < e->layers.size(); ++l) {
        const LkLayer& ly = e->layers[l];
        std::vector<const char*> need = {"norm1", "w_in", "w_o"};
        if (ly.c.ff_kind) need.insert(need.end(), {"norm2", "w_up", "w_down"});
        for (const char* n : need)
            if (!ly.w(n)) return set_error("asd_lukopel_forward: layer %d has no tensor %s", (int)l, n);
    }
    if (!tokens || !positions || !token_slot || !cu_q || !seq_slot || nseq <= 0 || max_qlen <= 0)
        return set_error("asd_lukopel_forward: bad index arguments");
    if (max_kv_len > e->max_pages * e->c.page_size)
        return set_error("asd_lukopel_forward: length bound %d exceeds the page table", max_kv_len);
    if (e->gw("pos") && e->c.max_positions > 0 && max_kv_len > e->c.max_positions)
        return set_error("asd_lukopel_forward: length bound %d exceeds the %d learned positions", max_kv_len,
                         e->c.max_positions);
    if (n_logit_rows > 0 && !logits_out) return set_error("asd_lukopel_forward: logits_out is NULL");
    if (n_logit_rows > e->c.max_tokens) return set_error("asd_lukopel_forward: too many logit rows");
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev != e->device) return set_error("asd_lukopel_forward: called on device %d, engine lives on %d", dev, e->device);
    const LkBatch b{SeqIndex{tokens, positions, token_slot, M}, cu_q, seq_slot, nseq, max_qlen, max_kv_len};
    return forward(e, b, logit_rows, logit_rows ? n_logit_rows : (n_logit_rows > 0 ? M : 0), logits_out, logits_ld,
                   layer_out, static_cast<cudaStream_t>(stream));
}

int asd_lukopel_profile_read(asd_lukopel_engine_t* h, float* ms_by_class, int* launches_by_class, int nclass) {
    LkEngine* e = static_cast<LkEngine*>(h);
    if (!e || !ms_by_class || nclass < LK_NCLASS) return set_error("asd_lukopel_profile_read: bad argument");
    ASD_CUDA(e->prof.read(ms_by_class, launches_by_class, nclass));
    return 0;
}

int asd_lukopel_device_error(asd_lukopel_engine_t* h) {
    LkEngine* e = static_cast<LkEngine*>(h);
    if (!e) return set_error("asd_lukopel_device_error: NULL engine");
    int v = 0;
    ASD_CUDA(cudaMemcpy(&v, e->dev_error, sizeof(int), cudaMemcpyDeviceToHost));
    if (v) return set_error("a Lukopel kernel gave up a bounded wait (tcgen05 linear)");
    return 0;
}

}  // extern "C"
