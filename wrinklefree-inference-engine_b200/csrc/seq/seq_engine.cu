// Serving engine for layer-stack sequence models (include/wf_seq.h): resident weights laid out for the kernels, a paged cache pool shared by
// all cached layers, fixed-size state slots (convolution tails, recurrent matrices), and the step function over a ragged batch of
// prompt portions and single decoded tokens.  The host side decides WHAT runs in a step (scheduler, trace replay); everything that
// computes is a kernel launched from here.
#include "seq_kernels.cuh"
#include "../pager.h"
#include "wf_seq.h"
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <algorithm>
#include <map>
#include <string>
#include <vector>

using namespace wf;
using namespace wf::seq;

namespace {

struct TensorSlot {
    std::string name;
    void* dst = nullptr;      // where the elements go (device)
    size_t count = 0;
    bool loaded = false;
};

struct LayerState {
    wf_seq_layer c;
    // weights (device, storage type)
    void *norm1, *norm2, *norm1b, *norm2b, *canon1, *canon2;
    void* wp = nullptr;       // fused input projections [np, W]
    int np = 0;
    void* wo = nullptr;       // [W, heads * vdim]
    // latent attention
    void *dkv_norm = nullptr, *uk = nullptr, *ukT = nullptr, *uv = nullptr;
    long long cache_off = 0;  // element offset of this layer inside a cache page
    // delta
    void *conv_w = nullptr, *A_log = nullptr, *dt_bias = nullptr, *onorm = nullptr;
    int C = 0;                // convolved channels
    // routed feed-forward
    void *router = nullptr, *correction = nullptr, *wgu = nullptr, *wd = nullptr;
    int nz = 0;               // rows of the router matrix: the experts, plus the shared expert's gate row when there is one
    // grouped-query attention: biases, column offsets of the parts inside the fused projection (-1: absent)
    void *qb = nullptr, *kb = nullptr, *vb = nullptr, *ob = nullptr;
    int k_off = -1, v_off = -1, g_off = -1;
    // one gated unit that every token runs: a dense feed-forward, or the shared expert of a routed one.  [gate | up] stacked, then down
    void *ugu = nullptr, *ud = nullptr;
    int uff = 0;
    float ulimit = 0.f;
    // attention: weights of the query / key norms, the bias table as loaded [rel_rows, heads] and expanded by distance (float [rel_n, heads])
    void *q_norm_w = nullptr, *k_norm_w = nullptr, *rel = nullptr;
    float* rel_dist = nullptr;
    int rel_n = 0;
    // recurrences: second factors of two-matrix projections (decay, gate), column offsets of the gate / write-strength / decay parts in the
    // fused projection; state-space: convolution bias, skip weights
    void *a2 = nullptr, *g2 = nullptr, *conv_b = nullptr, *Dskip = nullptr;
    int g_col = 0, b_col = 0, a_col = 0, n_decay = 0;
    int pair_state = 0;       // index of the second mixer's state in the engine's layer array
    // latent attention: query latent (norm weight, up-projection), learned sinks as loaded and as floats, rotation frequencies (double
    // [rope_dims / 2], tabulated at finalize) and the factor on cosines and sines; column of the [latent | rotated key] part in the projection
    void *dq_norm = nullptr, *uq = nullptr, *sink_raw = nullptr;
    float* sink_f = nullptr;
    double* freq = nullptr;
    float rope_mscale = 1.f;
    int kv_col = 0;
    // gated recurrences: the two gate biases (element-wise: z.b, x.b; matrix memory: i.b, f.b); state offset of the running maximum
    void *gb1 = nullptr, *gb2 = nullptr;
    size_t st_m = 0;
    // state slot offsets (floats)
    size_t st_canon1 = 0, st_canon2 = 0, st_conv = 0, st_S = 0;
};

}  // namespace

struct wf_seq_engine {
    wf_seq_config cfg;
    int dt = WF_BF16;
    size_t esz = 2;
    cudaStream_t stream = nullptr;
    std::vector<LayerState> layers;
    std::vector<TensorSlot> tensors;
    std::map<std::string, int> tensor_index;
    void *embed = nullptr, *final_norm = nullptr, *head = nullptr;
    bool finalized = false;
    // cache + state
    PageTable pt;
    std::vector<int32_t> h_len;       // [slots] tokens held
    void* pool = nullptr;
    long long page_stride = 0;        // elements per page
    float* state = nullptr;
    size_t slot_stride = 0;           // floats per slot
    int32_t* d_block_table = nullptr;
    // step metadata
    int32_t *h_meta = nullptr, *d_meta = nullptr;
    size_t meta_ints = 0;
    // workspace
    float *x = nullptr, *hn = nullptr, *y = nullptr, *proj = nullptr, *qr = nullptr, *qa = nullptr, *ov = nullptr, *qkvc = nullptr, *beta = nullptr,
          *decay = nullptr, *od = nullptr, *z = nullptr, *wts = nullptr, *gu = nullptr, *yexp = nullptr;
    void *hperm = nullptr, *h_t = nullptr, *qn = nullptr, *olat = nullptr, *og = nullptr, *hmid = nullptr, *xn = nullptr;
    float *gate = nullptr, *ugu = nullptr, *uy = nullptr;      // head gates; the every-token unit's [gate | up] rows and its output
    float *y2 = nullptr;              // output of the second mixer of a paired layer
    void* h_t2 = nullptr;             // WF_SEQ_BLOCK_PARALLEL: the feed-forward's input (second norm of the stream)
    float* qfull = nullptr;           // latent attention with a query latent: the up-projected queries
    void* cq = nullptr;               // ... and the normalised query latent
    float* mrun = nullptr;            // matrix memory: running maximum of the log gates per (token, head)
    float *gfull = nullptr, *afull = nullptr;   // recurrences: gate and decay logits when they are products of two matrices
    ScanWorkspace scan;               // state-space recurrence over long portions: per-chunk states (launch_delta_rule)
    void* uhmid = nullptr;
    int32_t *ids = nullptr, *counts = nullptr, *plan_scratch = nullptr, *sorted_rows = nullptr, *pair_row = nullptr, *tile_group = nullptr;
    int P = 0;                        // padded expert-row bound
    int fuse_input = 1;               // norm + input convolution (+ state roll of single-token sequences) in one kernel (WF_SEQ_FUSE_INPUT=0: three kernels)
    int attn_mma = 2;                 // latent attention on tensor cores where the sizes allow it: 2 keys-as-rows form first, 1 heads-as-rows form only, 0 plain kernel (WF_SEQ_ATTN_MMA)
    float* row_inv = nullptr;         // [max_step_tokens][norm groups] row statistics of the many-token input kernel
    int attn_waves = 4;               // decode attention: resident waves of CTAs the key splits aim at (WF_SEQ_ATTN_WAVES)
    float* gqa_ws = nullptr;          // partial results of key-split grouped-query attention: gqa_ws_rows (token, head, split) rows
    int gqa_ws_rows = 0;
    float* attn_ws = nullptr;         // partial results of key-split attention
    int attn_ws_rows = 0;             // token-splits it holds
    int pair_path_max = 64;           // up to this many (token, expert) pairs the experts run as per-pair weight streams (WF_SEQ_PAIR_MAX)
    float* logits = nullptr;
    size_t logits_rows = 0;
    float* d_uniform = nullptr;
    int32_t* d_next = nullptr;
    size_t sample_rows = 0;
    float* layer_tap = nullptr;
    // decode-only steps (one token per sequence) replay a CUDA graph captured per (sequences, wanted rows): their launch parameters depend
    // on nothing else.  A shape runs eagerly the first time (one-time kernel attributes are set then) and is captured the second time.
    int graph_max = 64;               // WF_SEQ_GRAPH_MAX: largest decode batch that is graphed (0: never)
    std::map<std::pair<int, int>, cudaGraphExec_t> graphs;
    std::map<std::pair<int, int>, int> graph_seen;
    // per-kernel-kind timing (wf_seq_profile_step): an event after every launch group; the time since the previous event goes to its label
    bool prof = false;
    std::vector<std::pair<const char*, cudaEvent_t>> marks;
    int launches = 0;
    size_t dev_bytes = 0;
    std::vector<void*> allocs;
};

namespace {

int dalloc_bytes(wf_seq_engine* e, void** p, size_t bytes) {
    void* q = nullptr;
    if (bytes == 0) bytes = 16;
    bytes = (bytes + 255) / 256 * 256;
    if (cuda_check(cudaMalloc(&q, bytes), "cudaMalloc")) return WF_ERR_CUDA;
    e->allocs.push_back(q);
    e->dev_bytes += bytes;
    *p = q;
    return WF_OK;
}
template <typename P>
int dalloc_t(wf_seq_engine* e, P** p, size_t count) { return dalloc_bytes(e, (void**)p, count * e->esz); }   // storage-type elements
template <typename P>
int dalloc_n(wf_seq_engine* e, P** p, size_t count) { return dalloc_bytes(e, (void**)p, count * sizeof(P)); }

void add_tensor(wf_seq_engine* e, const std::string& name, void* dst, size_t count) {
    TensorSlot t;
    t.name = name; t.dst = dst; t.count = count;
    e->tensor_index[name] = (int)e->tensors.size();
    e->tensors.push_back(t);
}
void* at(const wf_seq_engine* e, void* base, size_t elems) { return (char*)base + elems * e->esz; }

int validate(const wf_seq_config& c, const wf_seq_layer* L) {
    if (c.dtype != WF_SEQ_F32 && c.dtype != WF_SEQ_BF16) { set_error("wf_seq_create: dtype %d", c.dtype); return WF_ERR_INVALID; }
    if (c.vocab <= 0 || c.width <= 0 || c.n_layers <= 0 || c.norm_groups <= 0 || c.width % c.norm_groups || c.canon_taps < 1) {
        set_error("wf_seq_create: vocab %d width %d layers %d norm groups %d taps %d", c.vocab, c.width, c.n_layers, c.norm_groups, c.canon_taps);
        return WF_ERR_INVALID;
    }
    if (c.block_form != WF_SEQ_BLOCK_SANDWICH && c.block_form != WF_SEQ_BLOCK_POST && c.block_form != WF_SEQ_BLOCK_PARALLEL) { set_error("wf_seq_create: block form %d", c.block_form); return WF_ERR_INVALID; }
    if (c.page_size <= 0 || c.max_pages <= 0 || c.slots <= 0 || c.max_step_tokens <= 0) { set_error("wf_seq_create: page / slot / step sizes must be positive"); return WF_ERR_INVALID; }
    if (c.n_extra < 0) { set_error("wf_seq_create: %d extra mixers", c.n_extra); return WF_ERR_INVALID; }
    for (int i = 0; i < c.n_layers + c.n_extra; ++i) {
        const wf_seq_layer& l = L[i];
        if (l.heads <= 0 || l.dim <= 0 || l.vdim <= 0) { set_error("layer %d: heads / dim / vdim must be positive", i); return WF_ERR_INVALID; }
        if (i >= c.n_layers && (l.pair || l.has_ff || l.tied)) { set_error("mixer %d: a second mixer has no pair, feed-forward or tie of its own", i); return WF_ERR_INVALID; }
        if (l.pair && (l.pair < c.n_layers || l.pair >= c.n_layers + c.n_extra)) { set_error("layer %d: pair %d is not a second-mixer entry", i, l.pair); return WF_ERR_INVALID; }
        if (l.tied) {
            const wf_seq_layer* src = l.tied_to >= 0 && l.tied_to < c.n_layers && l.tied_to != i ? &L[l.tied_to] : nullptr;
            if (!src || src->tied || src->type != l.type || src->heads != l.heads || src->dim != l.dim || src->vdim != l.vdim || src->kv_heads != l.kv_heads ||
                src->has_ff != l.has_ff || src->ff != l.ff || (src->pair != 0) != (l.pair != 0) || src->conv != l.conv) {
                set_error("layer %d: tied_to %d must name another layer, with weights of its own and the same shape", i, l.tied_to); return WF_ERR_INVALID;
            }
            if (l.pair && (L[l.pair].type != L[src->pair].type || L[l.pair].heads != L[src->pair].heads || L[l.pair].dim != L[src->pair].dim ||
                           L[l.pair].vdim != L[src->pair].vdim || L[l.pair].kv_heads != L[src->pair].kv_heads || L[l.pair].conv != L[src->pair].conv)) {
                set_error("layer %d: its second mixer differs in shape from that of layer %d", i, l.tied_to); return WF_ERR_INVALID;
            }
        }
        if (l.type == WF_SEQ_LATENT_ATTENTION) {
            if (l.kv_rank <= 0 || l.rot_dim < 0 || l.window < 1 || l.rope_dims < 0 || l.rope_dims > l.rot_dim || (l.rope_dims & 1) || l.q_rank < 0) { set_error("layer %d: latent attention sizes", i); return WF_ERR_INVALID; }
            if (l.sink != 0 && l.sink != 2) { set_error("layer %d: latent attention takes no sink or a learned one per head", i); return WF_ERR_INVALID; }
            if (l.rope_factor < 0.f || (l.rope_factor > 0.f && !(l.rope_orig > 0.f && l.rope_fast > 0.f && l.rope_slow > 0.f && l.rope_base > 1.f))) { set_error("layer %d: frequency interpolation constants", i); return WF_ERR_INVALID; }
        } else if (l.type == WF_SEQ_MINGRU) {
            if (l.heads != 1 || l.dim != 1) { set_error("layer %d: the element-wise recurrence has heads = dim = 1 and vdim channels", i); return WF_ERR_INVALID; }
        } else if (l.type == WF_SEQ_MLSTM) {
            if (l.gate_cap < 0.f) { set_error("layer %d: gate cap %g", i, l.gate_cap); return WF_ERR_INVALID; }
        } else if (l.type == WF_SEQ_DELTA) {
            if (l.kv_heads <= 0 || l.heads % l.kv_heads || l.conv < 1 || l.decay_rank < 0 || l.gate_rank < 0) { set_error("layer %d: delta sizes", i); return WF_ERR_INVALID; }
        } else if (l.type == WF_SEQ_SSD) {
            if (l.kv_heads <= 0 || l.heads % l.kv_heads || l.conv < 1 || l.out_norm_groups < 1 || (l.heads * l.vdim) % l.out_norm_groups) { set_error("layer %d: state-space sizes", i); return WF_ERR_INVALID; }
        } else if (l.type == WF_SEQ_GQA_ATTENTION) {
            if (l.kv_heads <= 0 || l.heads % l.kv_heads || l.window < 1) { set_error("layer %d: attention sizes", i); return WF_ERR_INVALID; }
            if (l.v_is_k && (l.vdim != l.dim || l.v_norm || l.kv_from >= 0)) { set_error("layer %d: values that are the keys have the keys' size, no norm of their own and a cache of their own", i); return WF_ERR_INVALID; }
            if (l.sink < 0 || l.sink > 1) { set_error("layer %d: grouped-query attention takes no sink or the extra one", i); return WF_ERR_INVALID; }
            if (l.qk_norm < 0 || l.qk_norm > 3 || l.rope_dims < 0 || (l.rope_dims & 1) || l.rope_dims > l.dim || l.chunk < 0 || l.rel_rows < 0 || l.softcap < 0.f ||
                (l.rel_rows > 0 && (l.rel_rows < 2 || !(l.rel_far > (float)(l.rel_rows / 2)))) || l.head_gate < 0 || l.head_gate > 2 || l.proj_bias < 0 || l.proj_bias > 2) {
                set_error("layer %d: attention options", i); return WF_ERR_INVALID;
            }
            if (l.kv_from >= 0) {
                const wf_seq_layer* src = l.kv_from < i ? &L[l.kv_from] : nullptr;
                if (!src || src->type != WF_SEQ_GQA_ATTENTION || src->kv_from >= 0 || src->kv_heads != l.kv_heads || src->dim != l.dim || src->vdim != l.vdim) {
                    set_error("layer %d: kv_from %d must name an earlier attention layer with its own key / value projections and the same key / value sizes", i, l.kv_from);
                    return WF_ERR_INVALID;
                }
            }
        } else { set_error("layer %d: unknown mixer type %d", i, l.type); return WF_ERR_INVALID; }
        if (l.has_ff != WF_SEQ_FF_NONE && l.has_ff != WF_SEQ_FF_ROUTED && l.has_ff != WF_SEQ_FF_DENSE) { set_error("layer %d: feed-forward kind %d", i, l.has_ff); return WF_ERR_INVALID; }
        if (l.has_ff == WF_SEQ_FF_DENSE && l.ff <= 0) { set_error("layer %d: dense feed-forward size", i); return WF_ERR_INVALID; }
        if (l.ff_act == WF_SEQ_ACT_RELU2 && l.has_ff != WF_SEQ_FF_DENSE && l.has_ff != WF_SEQ_FF_NONE) { set_error("layer %d: the ungated activation belongs to a dense feed-forward", i); return WF_ERR_INVALID; }
        if (c.block_form == WF_SEQ_BLOCK_PARALLEL && l.has_ff == WF_SEQ_FF_ROUTED) { set_error("layer %d: the parallel block form takes a dense feed-forward or none", i); return WF_ERR_UNSUPPORTED; }
        if (l.has_ff && (l.ff_act < 0 || l.ff_act > 3 || l.shared_ff < 0)) { set_error("layer %d: feed-forward activation / shared size", i); return WF_ERR_INVALID; }
        if (l.has_ff == WF_SEQ_FF_ROUTED) {
            const int N = l.experts + l.identity;
            if (l.experts < 0 || l.identity < 0 || N <= 0 || l.top < 1 || l.top > N || l.groups < 1 || N % l.groups || l.keep < 1 || l.keep > l.groups || (l.experts > 0 && l.ff <= 0)) {
                set_error("layer %d: router sizes", i); return WF_ERR_INVALID;
            }
        }
    }
    return WF_OK;
}

void mark(wf_seq_engine* e, const char* label) {
    if (!e->prof) return;
    cudaEvent_t ev;
    cudaEventCreate(&ev);
    cudaEventRecord(ev, e->stream);
    e->marks.push_back({label, ev});
}

struct StepView {
    Batch b;
    const int32_t* tokens;
    const int32_t* want;
};

// host bookkeeping + one H2D copy of a step's index arrays
int prepare_step(wf_seq_engine* e, int nseq, const int32_t* slots, const int32_t* counts, const int32_t* tokens, int nwant, const int32_t* want,
                 StepView* v) {
    const wf_seq_config& c = e->cfg;
    if (!e->finalized) { set_error("wf_seq_step: weights are not finalized"); return WF_ERR_INVALID; }
    if (nseq <= 0 || nseq > c.slots) { set_error("wf_seq_step: %d sequences (slots: %d)", nseq, c.slots); return WF_ERR_INVALID; }
    int n = 0;
    for (int i = 0; i < nseq; ++i) {
        const int s = slots[i];
        if (s < 0 || s >= c.slots || !e->pt.live[s]) { set_error("wf_seq_step: slot %d is not live", s); return WF_ERR_INVALID; }
        for (int j = 0; j < i; ++j) if (slots[j] == s) { set_error("wf_seq_step: slot %d twice in one step", s); return WF_ERR_INVALID; }
        if (counts[i] <= 0) { set_error("wf_seq_step: sequence %d brings %d tokens", i, counts[i]); return WF_ERR_INVALID; }
        n += counts[i];
    }
    if (n > c.max_step_tokens) { set_error("wf_seq_step: %d tokens in one step (limit %d)", n, c.max_step_tokens); return WF_ERR_INVALID; }
    if (nwant < 0 || nwant > n) { set_error("wf_seq_step: %d wanted rows of %d tokens", nwant, n); return WF_ERR_INVALID; }
    for (int j = 0; j < nwant; ++j) if (want[j] < 0 || want[j] >= n) { set_error("wf_seq_step: wanted row %d out of range", want[j]); return WF_ERR_INVALID; }
    if (tokens) for (int i = 0; i < n; ++i) if (tokens[i] < 0 || tokens[i] >= c.vocab) { set_error("wf_seq_step: token id %d outside the vocabulary", tokens[i]); return WF_ERR_INVALID; }
    // pages for the new tokens (all or nothing)
    for (int i = 0; i < nseq; ++i) {
        if (!e->pt.ensure(slots[i], e->h_len[slots[i]] + counts[i])) {
            set_error("wf_seq_step: cache pool exhausted (%d pages of %d tokens, %d free)", c.max_pages, c.page_size, (int)e->pt.free_pages.size());
            for (int j = 0; j <= i; ++j) e->pt.truncate(slots[j], e->h_len[slots[j]]);
            return WF_ERR_INVALID;
        }
    }
    int32_t* m = e->h_meta;
    const size_t T = c.max_step_tokens, S = c.slots;
    int32_t *m_tok = m, *m_tseq = m + T, *m_tpos = m + 2 * T, *m_start = m + 3 * T, *m_len = m_start + S, *m_pos0 = m_len + S, *m_slot = m_pos0 + S,
            *m_want = m_slot + S;
    int at_ = 0;
    for (int i = 0; i < nseq; ++i) {
        m_start[i] = at_; m_len[i] = counts[i]; m_pos0[i] = e->h_len[slots[i]]; m_slot[i] = slots[i];
        for (int k = 0; k < counts[i]; ++k) { m_tok[at_] = tokens ? tokens[at_] : 0; m_tseq[at_] = i; m_tpos[at_] = m_pos0[i] + k; ++at_; }
    }
    for (int j = 0; j < nwant; ++j) m_want[j] = want[j];
    if (cuda_check(cudaMemcpyAsync(e->d_meta, m, e->meta_ints * 4, cudaMemcpyHostToDevice, e->stream), "step metadata H2D")) return WF_ERR_CUDA;
    if (e->pt.dirty) {
        std::vector<int32_t> tmp(e->pt.table);
        for (auto& p : tmp) if (p < 0) p = 0;      // a stale lookup can never leave the pool
        if (cuda_check(cudaMemcpyAsync(e->d_block_table, tmp.data(), tmp.size() * 4, cudaMemcpyHostToDevice, e->stream), "block table H2D")) return WF_ERR_CUDA;
        if (cuda_check(cudaStreamSynchronize(e->stream), "sync")) return WF_ERR_CUDA;   // tmp is pageable
        e->pt.dirty = false;
    }
    int32_t* d = e->d_meta;
    v->tokens = d;
    v->b.n = n; v->b.nseq = nseq;
    v->b.max_len = 0;
    for (int i = 0; i < nseq; ++i) v->b.max_len = std::max(v->b.max_len, (int)counts[i]);
    v->b.tok_seq = d + T; v->b.tok_pos = d + 2 * T;
    v->b.seq_start = d + 3 * T; v->b.seq_len = d + 3 * T + S; v->b.seq_pos0 = d + 3 * T + 2 * S; v->b.seq_slot = d + 3 * T + 3 * S;
    v->want = d + 3 * T + 4 * S;
    return WF_OK;
}

void commit_lengths(wf_seq_engine* e, int nseq, const int32_t* slots, const int32_t* counts) {
    for (int i = 0; i < nseq; ++i) e->h_len[slots[i]] += counts[i];
}

GemmArgs lin(const void* A, int a_f32, int lda, const void* B, int ldb, void* C, int c_f32, int ldc, int M, int N, int K) {
    GemmArgs g;
    g.A = A; g.a_f32 = a_f32; g.lda = lda; g.B = B; g.ldb = ldb; g.C = C; g.c_f32 = c_f32; g.ldc = ldc; g.M = M; g.N = N; g.K = K;
    return g;
}

// h (post-convolution input, storage type [n, W]) -> y float [n, W]
int run_latent(wf_seq_engine* e, LayerState& L, const Batch& b, float* out) {
    const wf_seq_layer& c = L.c;
    const int W = e->cfg.width, n = b.n, H = c.heads, per = c.dim + c.rot_dim, nq = H * per, nkv = c.kv_rank + c.rot_dim, nv = H * c.vdim;
    cudaStream_t s = e->stream;
    int rc;
    LatentDims D{H, c.dim, c.rot_dim, c.vdim, c.kv_rank, c.scale, c.rope_base, c.rope_dims, c.window};
    D.interleaved = c.rope_interleaved; D.freq = L.freq; D.mscale = L.rope_mscale; D.sink = L.sink_f;
    PagedCache pc{e->pool, e->page_stride, L.cache_off, e->cfg.page_size, e->d_block_table, e->pt.max_blocks};
    if ((rc = launch_gemm(e->dt, lin(e->h_t, 0, W, L.wp, W, e->proj, 1, L.np, n, L.np, W), s))) return rc;     // [q or its latent | dkv | g]
    mark(e, "latent.proj_gemm");
    const float* qsrc = e->proj;
    int ldq = L.np;
    if (c.q_rank > 0) {     // the queries' own latent: weighted RMS norm, then the up-projection
        if ((rc = launch_group_rmsnorm(e->dt, e->proj, L.np, L.dq_norm, 1, e->cfg.eps, n, c.q_rank, nullptr, nullptr, 0, e->cq, c.q_rank, nullptr, s))) return rc;
        if ((rc = launch_gemm(e->dt, lin(e->cq, 0, c.q_rank, L.uq, c.q_rank, e->qfull, 1, nq, n, nq, c.q_rank), s))) return rc;
        mark(e, "latent.query_latent");
        qsrc = e->qfull; ldq = nq;
    }
    if ((rc = launch_latent_q_prep(e->dt, b, D, qsrc, ldq, e->qn, e->qr, s))) return rc;
    if ((rc = launch_latent_kv_write(e->dt, b, D, e->proj + L.kv_col, L.np, L.dkv_norm, e->cfg.eps, pc, s))) return rc;
    mark(e, "latent.q_prep+kv_write");
    {   // qa[i, h, :] = W_uk[h]^T qn[i, h, :]
        GemmArgs g = lin(e->qn, 0, H * c.dim, L.ukT, c.dim, e->qa, 1, H * c.kv_rank, n, c.kv_rank, c.dim);
        g.batch = H; g.sA = c.dim; g.sB = (long long)c.kv_rank * c.dim; g.sC = c.kv_rank;
        if ((rc = launch_gemm(e->dt, g, s))) return rc;
        mark(e, "latent.absorb_gemm");
    }
    const bool rows_ok = L.cache_off % 8 == 0 && e->page_stride % 8 == 0;       // cached rows start 16-byte aligned
    const bool use_kt = e->dt == WF_BF16 && e->attn_mma >= 2 && rows_ok && latent_attn_kt_usable(D);
    const bool use_ht = e->dt == WF_BF16 && e->attn_mma >= 1 && rows_ok && !use_kt && latent_attn_mma_usable(D);
    if (use_kt || use_ht) {
        // few query tokens and a long window: split the keys so that one resident wave of CTAs covers the machine
        // (a CTA holds Q, two key tiles and P in shared memory: that decides how many are resident at once)
        int splits = 1;
        const int span = c.window < e->cfg.max_pages * e->cfg.page_size ? c.window : e->cfg.max_pages * e->cfg.page_size;
        const int resident = sm_count() * (use_kt ? latent_attn_kt_ctas_per_sm(D) : latent_attn_mma_ctas_per_sm(D));
        if (2 * n <= resident) {
            splits = resident / n;
            if (splits > span / 128) splits = span / 128;
            if (splits > e->attn_ws_rows / n) splits = e->attn_ws_rows / n;
            if (splits > 16) splits = 16;
            if (splits < 1) splits = 1;
        }
        if (use_kt) { if ((rc = launch_latent_attn_kt(b, D, e->qa, e->qr, pc, e->olat, e->attn_ws, splits, s))) return rc; }
        else if ((rc = launch_latent_attn_mma(b, D, e->qa, e->qr, pc, e->olat, e->attn_ws, splits, s))) return rc;
    } else if ((rc = launch_latent_attn(e->dt, b, D, e->qa, e->qr, pc, e->olat, s))) return rc;
    mark(e, "latent.attention");
    {   // ov[i, h, :] = W_uv[h] olat[i, h, :]
        GemmArgs g = lin(e->olat, 0, H * c.kv_rank, L.uv, c.kv_rank, e->ov, 1, nv, n, c.vdim, c.kv_rank);
        g.batch = H; g.sA = c.kv_rank; g.sB = (long long)c.vdim * c.kv_rank; g.sC = c.vdim;
        if ((rc = launch_gemm(e->dt, g, s))) return rc;
        mark(e, "latent.value_up_gemm");
    }
    // sigmoid gate per output element, or a plain conversion to the product operand
    if ((rc = launch_gate_mul(e->dt, e->ov, nv, c.head_gate ? e->proj + L.kv_col + nkv : e->ov, c.head_gate ? L.np : nv, c.head_gate ? 0 : 2, n, nv, e->og, nv, s))) return rc;
    mark(e, "latent.gate");
    rc = launch_gemm(e->dt, lin(e->og, 0, nv, L.wo, nv, out, 1, W, n, W, nv), s);
    mark(e, "latent.out_gemm");
    return rc;
}

int run_delta(wf_seq_engine* e, LayerState& L, const Batch& b, float* out) {
    const wf_seq_layer& c = L.c;
    const int W = e->cfg.width, n = b.n, H = c.heads, nv = H * c.vdim, C = L.C;
    cudaStream_t s = e->stream;
    int rc;
    DeltaDims D{H, c.kv_heads, c.dim, c.vdim};
    D.vec_decay = c.decay_channels ? 1 : 0;
    if ((rc = launch_gemm(e->dt, lin(e->h_t, 0, W, L.wp, W, e->proj, 1, L.np, n, L.np, W), s))) return rc;     // [q | k | v | g or g1 | b | a or a1]
    mark(e, "delta.proj_gemm");
    // gate and decay logits: columns of the fused projection, or a second small product on its low-rank columns
    const float* g_raw = e->proj + L.g_col;
    int ldg = L.np;
    if (c.gate_rank > 0) {
        if ((rc = launch_gemm(e->dt, lin(e->proj + L.g_col, 1, L.np, L.g2, c.gate_rank, e->gfull, 1, nv, n, nv, c.gate_rank), s))) return rc;
        g_raw = e->gfull; ldg = nv;
    }
    const float* a_raw = e->proj + L.a_col;
    int lda = L.np;
    if (c.decay_rank > 0) {
        if ((rc = launch_gemm(e->dt, lin(e->proj + L.a_col, 1, L.np, L.a2, c.decay_rank, e->afull, 1, L.n_decay, n, L.n_decay, c.decay_rank), s))) return rc;
        a_raw = e->afull; lda = L.n_decay;
    }
    if (c.gate_rank > 0 || c.decay_rank > 0) mark(e, "delta.lowrank_gemm");
    float* st_conv = e->state + L.st_conv;
    if ((rc = launch_causal_taps(e->dt, b, e->proj, L.np, L.conv_w, c.conv, C, st_conv, e->slot_stride, 0, 1, nullptr, 0, e->qkvc, C, s))) return rc;
    if ((rc = launch_taps_state(b, e->proj, L.np, c.conv, C, st_conv, e->slot_stride, s))) return rc;
    const float* b_raw = e->proj + L.b_col;
    if ((rc = launch_delta_prep(e->dt, D, n, e->qkvc, C, a_raw, lda, b_raw, L.np, L.A_log, L.dt_bias, e->beta, e->decay, s))) return rc;
    mark(e, "delta.conv+prep");
    if ((rc = launch_delta_rule(b, D, e->qkvc, C, e->beta, e->decay, e->state + L.st_S, e->slot_stride, e->od, s))) return rc;
    mark(e, "delta.rule");
    if ((rc = launch_delta_post(e->dt, D, n, e->od, L.onorm, e->cfg.eps, g_raw, ldg, e->og, s, c.gate_act))) return rc;
    mark(e, "delta.post");
    rc = launch_gemm(e->dt, lin(e->og, 0, nv, L.wo, nv, out, 1, W, n, W, nv), s);
    mark(e, "delta.out_gemm");
    return rc;
}

// state-space recurrence: [z | x | B | C | dt] projection -> convolution + silu over x | B | C -> step sizes and decays -> the recurrence
// (the delta-rule kernel without its correction: key = B, query = C, value = x, write strength = dt) -> skip, gate, grouped norm -> output
int run_ssd(wf_seq_engine* e, LayerState& L, const Batch& b, float* out) {
    const wf_seq_layer& c = L.c;
    const int W = e->cfg.width, n = b.n, H = c.heads, inner = H * c.vdim, GN = c.kv_heads * c.dim, C = L.C;
    cudaStream_t s = e->stream;
    int rc;
    if ((rc = launch_gemm(e->dt, lin(e->h_t, 0, W, L.wp, W, e->proj, 1, L.np, n, L.np, W), s))) return rc;
    mark(e, "ssd.proj_gemm");
    float* st_conv = e->state + L.st_conv;
    const float* xbc_raw = e->proj + inner;
    if ((rc = launch_causal_taps(e->dt, b, xbc_raw, L.np, L.conv_w, c.conv, C, st_conv, e->slot_stride, 0, 1, nullptr, 0, e->qkvc, C, s, L.conv_b))) return rc;
    if ((rc = launch_taps_state(b, xbc_raw, L.np, c.conv, C, st_conv, e->slot_stride, s))) return rc;
    if ((rc = launch_ssd_prep(e->dt, n, H, e->proj + 2 * inner + 2 * GN, L.np, L.A_log, L.dt_bias, e->beta, e->decay, s))) return rc;
    mark(e, "ssd.conv+prep");
    DeltaDims D{H, c.kv_heads, c.dim, c.vdim};
    D.no_delta = 1; D.v_off = 0; D.k_off = inner; D.q_off = inner + GN;
    if ((rc = launch_delta_rule(b, D, e->qkvc, C, e->beta, e->decay, e->state + L.st_S, e->slot_stride, e->od, s, &e->scan))) return rc;
    mark(e, "ssd.recurrence");
    if ((rc = launch_ssd_post(e->dt, n, H, c.vdim, c.out_norm_groups, e->od, e->qkvc, C, e->proj, L.np, L.Dskip, L.onorm, e->cfg.eps, e->og, s))) return rc;
    mark(e, "ssd.post");
    rc = launch_gemm(e->dt, lin(e->og, 0, inner, L.wo, inner, out, 1, W, n, W, inner), s);
    mark(e, "ssd.out_gemm");
    return rc;
}

// h_t -> y float [n, W].  In the post form the output projection's bias is NOT added here: the norm kernel that follows takes it
int run_gqa(wf_seq_engine* e, LayerState& L, const Batch& b, float* out) {
    const wf_seq_layer& c = L.c;
    const int W = e->cfg.width, n = b.n, nv = c.heads * c.vdim;
    cudaStream_t s = e->stream;
    int rc;
    GqaDims D{c.heads, c.kv_heads, c.dim, c.vdim, c.scale, c.dist_exp, c.window, c.qk_norm, c.v_norm};
    D.rope_dims = c.rope_dims; D.rope_interleaved = c.rope_interleaved; D.rope_base = c.rope_base;
    D.q_norm_w = L.q_norm_w; D.k_norm_w = L.k_norm_w;
    D.chunk = c.chunk; D.sink = c.sink; D.gate_elem = c.head_gate == 2; D.softcap = c.softcap;
    D.rel = L.rel_dist; D.rel_n = L.rel_n; D.v_is_k = c.v_is_k;
    const LayerState& src = c.kv_from >= 0 ? e->layers[c.kv_from] : L;        // whose cache rows this layer reads
    PagedCache pc{e->pool, e->page_stride, src.cache_off, e->cfg.page_size, e->d_block_table, e->pt.max_blocks};
    if ((rc = launch_gemm(e->dt, lin(e->h_t, 0, W, L.wp, W, e->proj, 1, L.np, n, L.np, W), s))) return rc;     // [q | k | v | g]
    mark(e, "attn.proj_gemm");
    if ((rc = launch_gqa_prep(e->dt, b, D, e->proj, L.np, L.k_off, L.v_off, L.g_off, L.qb, L.kb, L.vb, e->cfg.eps, pc, e->qn, c.head_gate ? e->gate : nullptr, s))) return rc;
    mark(e, "attn.prep+kv_write");
    const float* gate = c.head_gate ? e->gate : nullptr;
    if (e->dt == WF_BF16 && e->attn_mma >= 1 && gqa_attn_mma_usable(D, pc) && gqa_attn_mma_takes(D)) {
        // decoding (one token per sequence): few CTAs with long key ranges, so the keys are cut until there are about four resident
        // waves of CTAs (two are resident per SM): the machine is covered and the last wave's tail stays short.
        // The cut depends on the batch size and the pool only, never on the lengths: a captured step stays valid.
        int splits = 1;
        if (n == b.nseq) {
            long long span = std::min<long long>(c.window, (long long)e->cfg.max_pages * e->cfg.page_size);
            if (c.chunk > 0 && c.chunk < span) span = c.chunk;
            const int ctas = n * c.kv_heads, resident = 2 * sm_count();
            splits = (e->attn_waves * resident + ctas - 1) / ctas;
            if (splits > span / 256) splits = (int)(span / 256);
            if (splits > e->gqa_ws_rows / (n * c.heads)) splits = e->gqa_ws_rows / (n * c.heads);
            if (splits > 16) splits = 16;
            if (splits < 1) splits = 1;
        }
        if ((rc = launch_gqa_attn_mma(b, D, e->qn, gate, pc, e->og, e->gqa_ws, splits, s))) return rc;
    } else if ((rc = launch_gqa_attn(e->dt, b, D, e->qn, gate, pc, e->og, s))) return rc;
    mark(e, D.softcap > 0.f || D.rel ? "attn.attention(cap+bias)" : "attn.attention");
    rc = launch_gemm(e->dt, lin(e->og, 0, nv, L.wo, nv, out, 1, W, n, W, nv), s);
    // the single-gain norm of the post form takes the bias itself, except for paired mixers (their outputs are combined first)
    if (!rc && L.ob && !(e->cfg.block_form == WF_SEQ_BLOCK_POST && !e->cfg.norm_weights && !L.c.pair && out == e->y)) rc = launch_add_bias(e->dt, out, W, L.ob, n, W, s);
    mark(e, "attn.out_gemm");
    return rc;
}

// element-wise gated recurrence: [z | x | g] projection -> the recurrence over the portion (gate, candidate, state, silu read-out) -> output
int run_mingru(wf_seq_engine* e, LayerState& L, const Batch& b, float* out) {
    const int W = e->cfg.width, n = b.n, C = L.c.vdim;
    cudaStream_t s = e->stream;
    int rc;
    if ((rc = launch_gemm(e->dt, lin(e->h_t, 0, W, L.wp, W, e->proj, 1, L.np, n, L.np, W), s))) return rc;
    mark(e, "mingru.proj_gemm");
    if ((rc = launch_mingru(e->dt, b, C, e->proj, L.np, 0, C, 2 * C, L.gb1, L.gb2, e->state + L.st_S, e->slot_stride, e->og, s))) return rc;
    mark(e, "mingru.recurrence");
    rc = launch_gemm(e->dt, lin(e->og, 0, C, L.wo, C, out, 1, W, n, W, C), s);
    mark(e, "mingru.out_gemm");
    return rc;
}

// matrix memory: [q | k | v | g | i | f] projection -> log gates, running maximum, keep / put factors -> the plain decayed outer-product
// recurrence with the normaliser as one more value column -> division, per-head norm, weight, sigmoid gate -> output
int run_mlstm(wf_seq_engine* e, LayerState& L, const Batch& b, float* out) {
    const wf_seq_layer& c = L.c;
    const int W = e->cfg.width, n = b.n, H = c.heads, nk = H * c.dim, nv = H * c.vdim;
    cudaStream_t s = e->stream;
    int rc;
    if ((rc = launch_gemm(e->dt, lin(e->h_t, 0, W, L.wp, W, e->proj, 1, L.np, n, L.np, W), s))) return rc;
    mark(e, "mlstm.proj_gemm");
    if ((rc = launch_mlstm_gates(e->dt, b, H, e->proj, L.np, 2 * nk + 2 * nv, 2 * nk + 2 * nv + H, L.gb1, L.gb2, c.gate_cap, e->state + L.st_m, e->slot_stride,
                                 e->decay, e->beta, e->mrun, s))) return rc;
    mark(e, "mlstm.gates");
    DeltaDims D{H, H, c.dim, c.vdim};
    D.no_delta = 1; D.ones_col = 1; D.q_off = 0; D.k_off = nk; D.v_off = 2 * nk;
    if ((rc = launch_delta_rule(b, D, e->proj, L.np, e->beta, e->decay, e->state + L.st_S, e->slot_stride, e->od, s, &e->scan))) return rc;
    mark(e, "mlstm.recurrence");
    if ((rc = launch_mlstm_post(e->dt, n, H, c.vdim, e->od, e->mrun, 1.f / sqrtf((float)c.dim), L.onorm, e->cfg.eps, e->proj + 2 * nk + nv, L.np, e->og, s))) return rc;
    mark(e, "mlstm.post");
    rc = launch_gemm(e->dt, lin(e->og, 0, nv, L.wo, nv, out, 1, W, n, W, nv), s);
    mark(e, "mlstm.out_gemm");
    return rc;
}

int run_one_mixer(wf_seq_engine* e, LayerState& L, const Batch& b, float* out) {
    switch (L.c.type) {
        case WF_SEQ_MINGRU: return run_mingru(e, L, b, out);
        case WF_SEQ_MLSTM: return run_mlstm(e, L, b, out);
        case WF_SEQ_GQA_ATTENTION: return run_gqa(e, L, b, out);
        case WF_SEQ_LATENT_ATTENTION: return run_latent(e, L, b, out);
        case WF_SEQ_SSD: return run_ssd(e, L, b, out);
        default: return run_delta(e, L, b, out);
    }
}

// h_t -> y.  A paired layer runs its two mixers one after the other on the same input (they share the projection workspaces); their
// outputs are combined in float, here or (combine = false) by the norm kernel that follows.
int run_mixer(wf_seq_engine* e, LayerState& L, const Batch& b, bool combine = true) {
    int rc;
    if ((rc = run_one_mixer(e, L, b, e->y))) return rc;
    if (!L.c.pair) return WF_OK;
    if ((rc = run_one_mixer(e, e->layers[L.pair_state], b, e->y2))) return rc;
    if (!combine) return WF_OK;                  // the caller's norm kernel forms mix_scale * y + pair_scale * y2 on its way in
    rc = launch_axpby(e->y, L.c.mix_scale, e->y2, L.c.pair_scale, (size_t)b.n * e->cfg.width, e->stream);
    mark(e, "pair.combine");
    return rc;
}

// the gated unit every token runs (dense feed-forward / shared expert): h_t -> out float [n, W]
int run_unit(wf_seq_engine* e, LayerState& L, const Batch& b, float* out, const void* in = nullptr) {
    const int W = e->cfg.width, n = b.n, ff = L.uff;
    cudaStream_t s = e->stream;
    int rc;
    if (!in) in = e->h_t;
    const int nu = L.c.ff_act == WF_SEQ_ACT_RELU2 ? ff : 2 * ff;       // the ungated activation has no gate half
    if ((rc = launch_gemm(e->dt, lin(in, 0, W, L.ugu, W, e->ugu, 1, nu, n, nu, W), s))) return rc;
    mark(e, "unit.gate_up");
    if ((rc = launch_silu_mul(e->dt, e->ugu, n, ff, nullptr, e->uhmid, s, L.c.ff_act, L.ulimit))) return rc;
    mark(e, "unit.act");
    rc = launch_gemm(e->dt, lin(e->uhmid, 0, ff, L.ud, ff, out, 1, W, n, W, ff), s);
    mark(e, "unit.down");
    return rc;
}

int run_ff(wf_seq_engine* e, LayerState& L, const Batch& b) {
    const wf_seq_layer& c = L.c;
    const int W = e->cfg.width, n = b.n, N = L.nz;
    cudaStream_t s = e->stream;
    int rc;
    if (c.has_ff == WF_SEQ_FF_DENSE) return run_unit(e, L, b, e->y);
    RouterDims R{c.experts, c.identity, c.top, c.groups, c.keep};
    R.act = c.router_act; R.group_top = c.group_top; R.norm = c.router_norm; R.scale = c.router_scale != 0.f ? c.router_scale : 1.f;   // a zeroed struct means unscaled
    // In the post form the sublayer's input IS the float stream, so the router reads it unrounded and multiplies in float — a router is
    // a 32-bit quantity, and a score that the rounding of its input moved across a neighbour's would change the chosen experts — and the
    // product and the choice are one kernel.  The sandwich form's input exists only in the storage type: product, then choice.
    const bool fused_router = e->cfg.block_form == WF_SEQ_BLOCK_POST && router_fused_usable(R, N, W);
    if (!fused_router) {
        GemmArgs g = e->cfg.block_form == WF_SEQ_BLOCK_POST ? lin(e->x, 1, W, L.router, W, e->z, 1, N, n, N, W) : lin(e->h_t, 0, W, L.router, W, e->z, 1, N, n, N, W);
        if (e->cfg.block_form == WF_SEQ_BLOCK_POST && (n > 8 || W % 8)) g.algo = 1;      // up to 8 aligned rows take the few-row stream, which multiplies in float too
        if ((rc = launch_gemm(e->dt, g, s))) return rc;     // expert logits [| shared gate logit]
        mark(e, "moe.router");
    }
    const float* sh_y = nullptr;
    const float* sh_gate = nullptr;
    if (c.shared_ff > 0) {
        if ((rc = run_unit(e, L, b, e->uy))) return rc;
        sh_y = e->uy; sh_gate = e->z + c.experts + c.identity;
    }
    const int pairs = n * c.top;
    GemmArgs gp = lin(e->h_t, 0, W, L.wgu, W, e->gu, 1, 2 * c.ff, pairs, 2 * c.ff, W);
    gp.group_stride = (long long)2 * c.ff * W;
    GemmArgs gd = lin(e->hmid, 0, c.ff, L.wd, c.ff, e->yexp, 1, W, pairs, W, c.ff);
    gd.group_stride = (long long)W * c.ff;
    const bool pair_path = c.experts > 0 && pairs <= e->pair_path_max && gemv_pairs_usable(e->dt, gp) && gemv_pairs_usable(e->dt, gd);
    // per-expert token counts are only needed to sort the pairs (the per-pair path sorts nothing)
    if (c.experts > 0 && !pair_path && cuda_check(cudaMemsetAsync(e->counts, 0, (size_t)c.experts * 4, s), "counts")) return WF_ERR_CUDA;
    if (fused_router) rc = launch_router_fused(e->dt, R, n, e->x, W, L.router, N, W, e->z, N, L.correction, e->ids, e->wts, pair_path ? nullptr : e->counts, s);
    else rc = launch_moe_route(e->dt, R, n, e->z, N, L.correction, e->ids, e->wts, pair_path ? nullptr : e->counts, s);
    if (rc) return rc;
    mark(e, "moe.router");
    if (pair_path) {
        // few tokens (decoding): one weight-streaming product per (token, expert) pair, no sorting
        if ((rc = launch_gemv_pairs(e->dt, gp, e->ids, c.experts, pairs, c.top, s))) return rc;
        mark(e, "moe.gate_up");
        if ((rc = launch_silu_mul(e->dt, e->gu, pairs, c.ff, nullptr, e->hmid, s, c.ff_act, c.ff_limit))) return rc;
        mark(e, "moe.silu_mul");
        if ((rc = launch_gemv_pairs(e->dt, gd, e->ids, c.experts, pairs, 1, s))) return rc;
        mark(e, "moe.down");
        rc = launch_moe_combine(e->dt, R, n, W, e->ids, e->wts, nullptr, e->yexp, e->h_t, e->y, s, sh_y, sh_gate, N);
        mark(e, "moe.combine");
        return rc;
    }
    if (c.experts > 0) {
        const int P = (n * c.top + GEMM_BM - 1) / GEMM_BM * GEMM_BM + c.experts * GEMM_BM;
        if ((rc = launch_moe_plan(R, n, e->ids, e->counts, e->plan_scratch, e->sorted_rows, e->pair_row, e->tile_group, P, s))) return rc;
        mark(e, "moe.plan");
        // the experts' input rows, expert after expert (a dense operand for the tensor-core product)
        if ((rc = launch_gather_rows(e->dt, e->h_t, W, e->sorted_rows, P, W, e->hperm, s))) return rc;
        GemmArgs g = lin(e->hperm, 0, W, L.wgu, W, e->gu, 1, 2 * c.ff, P, 2 * c.ff, W);
        g.tile_group = e->tile_group; g.group_stride = (long long)2 * c.ff * W; g.n_groups = c.experts;
        if ((rc = launch_gemm(e->dt, g, s))) return rc;
        mark(e, "moe.gate_up");
        if ((rc = launch_silu_mul(e->dt, e->gu, P, c.ff, e->tile_group, e->hmid, s, c.ff_act, c.ff_limit))) return rc;
        mark(e, "moe.silu_mul");
        GemmArgs g2 = lin(e->hmid, 0, c.ff, L.wd, c.ff, e->yexp, 1, W, P, W, c.ff);
        g2.tile_group = e->tile_group; g2.group_stride = (long long)W * c.ff; g2.n_groups = c.experts;
        if ((rc = launch_gemm(e->dt, g2, s))) return rc;
        mark(e, "moe.down");
    }
    rc = launch_moe_combine(e->dt, R, n, W, e->ids, e->wts, e->pair_row, e->yexp, e->h_t, e->y, s, sh_y, sh_gate, N);
    mark(e, "moe.combine");
    return rc;
}

// norm -> input convolution (state rolled forward) -> e->h_t
int run_input(wf_seq_engine* e, const Batch& b, const void* norm_w, const void* canon_w, size_t st_off) {
    const int W = e->cfg.width;
    cudaStream_t s = e->stream;
    int rc;
    if (e->fuse_input && b.n >= 64) {
        // many tokens: per-row statistics once, then a fully parallel apply (the one-block-per-token kernel recomputes them per tap)
        if ((rc = launch_norm_taps_rows(e->dt, b, e->x, W, norm_w, e->cfg.norm_groups, e->cfg.eps, canon_w, e->cfg.canon_taps, W, e->state + st_off, e->slot_stride,
                                        e->h_t, W, e->hn, e->row_inv, s))) return rc;
        rc = launch_taps_state(b, e->hn, W, e->cfg.canon_taps, W, e->state + st_off, e->slot_stride, s);
    } else if (e->fuse_input && norm_taps_usable(e->cfg.norm_groups, e->cfg.canon_taps, W)) {
        if ((rc = launch_norm_taps(e->dt, b, e->x, W, norm_w, e->cfg.norm_groups, e->cfg.eps, canon_w, e->cfg.canon_taps, W, e->state + st_off, e->slot_stride,
                                   e->h_t, W, e->hn, s))) return rc;
        rc = b.n == b.nseq ? WF_OK : launch_taps_state(b, e->hn, W, e->cfg.canon_taps, W, e->state + st_off, e->slot_stride, s, 1);
    } else {
        if ((rc = launch_group_rmsnorm(e->dt, e->x, W, norm_w, e->cfg.norm_groups, e->cfg.eps, b.n, W, nullptr, e->hn, W, nullptr, 0, nullptr, s))) return rc;
        if ((rc = launch_causal_taps(e->dt, b, e->hn, W, canon_w, e->cfg.canon_taps, W, e->state + st_off, e->slot_stride, 1, 0, e->h_t, W, nullptr, 0, s))) return rc;
        rc = launch_taps_state(b, e->hn, W, e->cfg.canon_taps, W, e->state + st_off, e->slot_stride, s);
    }
    mark(e, "norm+input_conv");
    return rc;
}

// WF_SEQ_BLOCK_POST: every sublayer reads the stream itself (h_t is its storage-type copy, refreshed by the kernel that updates the stream)
// and its output is normalised with one gain, scaled and added.
int run_layers_post(wf_seq_engine* e, const StepView& v) {
    const int W = e->cfg.width, n = v.b.n;
    const float mult = e->cfg.residual_mult, eps = e->cfg.eps;
    cudaStream_t s = e->stream;
    int rc;
    const float escale = e->cfg.embed_scale != 0.f ? e->cfg.embed_scale : 1.f;
    const bool vec = e->cfg.norm_weights != 0;            // weight vectors (one launch of the grouped norm with one group) or single gains
    if (e->cfg.pos_embed) { if ((rc = launch_embed_pos(e->dt, e->embed, v.tokens, v.b.tok_pos, n, W, e->cfg.pos_base, e->x, e->h_t, s))) return rc; }
    else if ((rc = launch_embed_f32(e->dt, e->embed, v.tokens, n, W, e->x, s, escale, e->h_t))) return rc;
    mark(e, "embed");
    for (int li = 0; li < e->cfg.n_layers; ++li) {
        LayerState& L = e->layers[li];
        if ((rc = run_mixer(e, L, v.b, !vec))) return rc;
        if (vec) rc = launch_group_rmsnorm(e->dt, e->y, W, L.norm1, 1, eps, n, W, e->x, e->x, W, e->h_t, W, nullptr, s, L.c.pair ? e->y2 : nullptr, L.c.mix_scale, L.c.pair_scale);
        else rc = launch_scalar_rmsnorm(e->dt, e->y, W, L.c.pair ? nullptr : L.ob, L.norm1, mult, eps, n, W, e->x, e->x, W, e->h_t, W, nullptr, s);
        if (rc) return rc;
        mark(e, "norm+residual");
        if (L.c.has_ff) {
            if ((rc = run_ff(e, L, v.b))) return rc;
            if (vec) rc = launch_group_rmsnorm(e->dt, e->y, W, L.norm2, 1, eps, n, W, e->x, e->x, W, e->h_t, W, nullptr, s);
            else rc = launch_scalar_rmsnorm(e->dt, e->y, W, nullptr, L.norm2, mult, eps, n, W, e->x, e->x, W, e->h_t, W, nullptr, s);
            if (rc) return rc;
            mark(e, "norm+residual");
        }
        if (e->layer_tap) {
            if (cuda_check(cudaMemcpyAsync(e->layer_tap + (size_t)li * n * W, e->x, (size_t)n * W * 4, cudaMemcpyDeviceToHost, s), "layer tap")) return WF_ERR_CUDA;
        }
    }
    return WF_OK;
}

// WF_SEQ_BLOCK_PARALLEL: the mixer and the feed-forward of a layer read the same stream, each through its own weighted norm, and the
// stream takes the sum of both.  One kernel per layer boundary adds the finished layer's outputs to the stream and forms the next layer's
// two norm outputs from one pass over the row (the two norms share their statistics).
int run_layers_parallel(wf_seq_engine* e, const StepView& v) {
    const int W = e->cfg.width, n = v.b.n, NL = e->cfg.n_layers;
    const float eps = e->cfg.eps, off = e->cfg.norm_offset;
    cudaStream_t s = e->stream;
    int rc;
    const float escale = e->cfg.embed_scale != 0.f ? e->cfg.embed_scale : 1.f;
    if ((rc = launch_embed_f32(e->dt, e->embed, v.tokens, n, W, e->x, s, escale))) return rc;
    mark(e, "embed");
    {
        LayerState& L0 = e->layers[0];
        if ((rc = launch_add_dual_norm(e->dt, e->x, nullptr, 0.f, nullptr, 0.f, nullptr, L0.norm1, L0.c.has_ff ? L0.norm2 : nullptr, off, eps, n, W, e->h_t, e->h_t2, s))) return rc;
        mark(e, "residual+norms");
    }
    for (int li = 0; li < NL; ++li) {
        LayerState& L = e->layers[li];
        if ((rc = run_mixer(e, L, v.b, false))) return rc;
        if (L.c.has_ff && (rc = run_unit(e, L, v.b, e->uy, e->h_t2))) return rc;
        LayerState* N = li + 1 < NL ? &e->layers[li + 1] : nullptr;
        if ((rc = launch_add_dual_norm(e->dt, e->x, e->y, L.c.pair ? L.c.mix_scale : 1.f, L.c.pair ? e->y2 : nullptr, L.c.pair_scale, L.c.has_ff ? e->uy : nullptr,
                                       N ? N->norm1 : nullptr, N && N->c.has_ff ? N->norm2 : nullptr, off, eps, n, W, e->h_t, e->h_t2, s))) return rc;
        mark(e, "residual+norms");
        if (e->layer_tap) {
            if (cuda_check(cudaMemcpyAsync(e->layer_tap + (size_t)li * n * W, e->x, (size_t)n * W * 4, cudaMemcpyDeviceToHost, s), "layer tap")) return WF_ERR_CUDA;
        }
    }
    return WF_OK;
}

int run_layers(wf_seq_engine* e, const StepView& v) {
    if (e->cfg.block_form == WF_SEQ_BLOCK_POST) return run_layers_post(e, v);
    if (e->cfg.block_form == WF_SEQ_BLOCK_PARALLEL) return run_layers_parallel(e, v);
    const int W = e->cfg.width, n = v.b.n;
    cudaStream_t s = e->stream;
    int rc;
    if ((rc = launch_embed_f32(e->dt, e->embed, v.tokens, n, W, e->x, s))) return rc;
    mark(e, "embed");
    for (int li = 0; li < e->cfg.n_layers; ++li) {
        LayerState& L = e->layers[li];
        if ((rc = run_input(e, v.b, L.norm1, L.canon1, L.st_canon1))) return rc;
        if ((rc = run_mixer(e, L, v.b))) return rc;
        if ((rc = launch_group_rmsnorm(e->dt, e->y, W, L.norm1b, e->cfg.norm_groups, e->cfg.eps, n, W, e->x, e->x, W, nullptr, 0, nullptr, s))) return rc;
        mark(e, "norm+residual");
        if (L.c.has_ff) {
            if ((rc = run_input(e, v.b, L.norm2, L.canon2, L.st_canon2))) return rc;
            if ((rc = run_ff(e, L, v.b))) return rc;
            if ((rc = launch_group_rmsnorm(e->dt, e->y, W, L.norm2b, e->cfg.norm_groups, e->cfg.eps, n, W, e->x, e->x, W, nullptr, 0, nullptr, s))) return rc;
            mark(e, "norm+residual");
        }
        if (e->layer_tap) {
            if (cuda_check(cudaMemcpyAsync(e->layer_tap + (size_t)li * n * W, e->x, (size_t)n * W * 4, cudaMemcpyDeviceToHost, s), "layer tap")) return WF_ERR_CUDA;
        }
    }
    return WF_OK;
}

int ensure_logits(wf_seq_engine* e, size_t rows) {
    if (rows <= e->logits_rows) return WF_OK;
    for (auto& g : e->graphs) cudaGraphExecDestroy(g.second);      // captured steps hold the old buffer's address
    e->graphs.clear();
    if (e->logits) { cudaFree(e->logits); e->dev_bytes -= e->logits_rows * e->cfg.vocab * 4; }
    e->logits = nullptr; e->logits_rows = 0;
    if (cuda_check(cudaMalloc((void**)&e->logits, rows * e->cfg.vocab * 4), "cudaMalloc logits")) return WF_ERR_CUDA;
    e->logits_rows = rows;
    e->dev_bytes += rows * e->cfg.vocab * 4;
    return WF_OK;
}

int run_head(wf_seq_engine* e, const StepView& v, int nwant) {
    if (nwant <= 0) return WF_OK;
    const int W = e->cfg.width;
    int rc;
    if ((rc = ensure_logits(e, nwant))) return rc;
    if (e->cfg.block_form == WF_SEQ_BLOCK_PARALLEL) rc = launch_group_rmsnorm(e->dt, e->x, W, e->final_norm, 1, e->cfg.eps, nwant, W, nullptr, nullptr, W, e->xn, W, v.want, e->stream, nullptr, 1.f, 0.f, e->cfg.norm_offset);
    else if (e->cfg.block_form == WF_SEQ_BLOCK_POST && e->cfg.norm_weights) rc = launch_group_rmsnorm(e->dt, e->x, W, e->final_norm, 1, e->cfg.eps, nwant, W, nullptr, nullptr, W, e->xn, W, v.want, e->stream);
    else if (e->cfg.block_form == WF_SEQ_BLOCK_POST) rc = launch_scalar_rmsnorm(e->dt, e->x, W, nullptr, e->final_norm, 1.f, e->cfg.eps, nwant, W, nullptr, nullptr, W, e->xn, W, v.want, e->stream);
    else rc = launch_group_rmsnorm(e->dt, e->x, W, e->final_norm, e->cfg.norm_groups, e->cfg.eps, nwant, W, nullptr, nullptr, W, e->xn, W, v.want, e->stream);
    if (rc) return rc;
    rc = launch_gemm(e->dt, lin(e->xn, 0, W, e->head, W, e->logits, 1, e->cfg.vocab, nwant, e->cfg.vocab, W), e->stream);
    mark(e, "final_norm+head_gemm");
    return rc;
}

// layers + head of one step: eagerly, or (decode-only shapes seen before) as a captured graph
int run_model(wf_seq_engine* e, const StepView& v, int nwant) {
    int rc;
    const bool decode_only = v.b.n == v.b.nseq;
    if (!decode_only || v.b.n > e->graph_max || e->layer_tap || e->prof) {
        if ((rc = run_layers(e, v))) return rc;
        return run_head(e, v, nwant);
    }
    if ((rc = ensure_logits(e, nwant))) return rc;
    const std::pair<int, int> key(v.b.n, nwant);
    auto it = e->graphs.find(key);
    if (it == e->graphs.end()) {
        if (e->graph_seen[key]++ == 0) {
            if ((rc = run_layers(e, v))) return rc;
            return run_head(e, v, nwant);
        }
        if (cuda_check(cudaStreamBeginCapture(e->stream, cudaStreamCaptureModeThreadLocal), "begin capture")) return WF_ERR_CUDA;
        rc = run_layers(e, v);
        if (!rc) rc = run_head(e, v, nwant);
        cudaGraph_t graph = nullptr;
        const cudaError_t ce = cudaStreamEndCapture(e->stream, &graph);
        if (rc) { if (graph) cudaGraphDestroy(graph); return rc; }
        if (cuda_check(ce, "end capture")) return WF_ERR_CUDA;
        cudaGraphExec_t exec = nullptr;
        const cudaError_t ie = cudaGraphInstantiate(&exec, graph, 0);
        cudaGraphDestroy(graph);
        if (cuda_check(ie, "graph instantiate")) return WF_ERR_CUDA;
        it = e->graphs.emplace(key, exec).first;
    }
    return cuda_check(cudaGraphLaunch(it->second, e->stream), "graph launch");
}

}  // namespace

extern "C" int wf_seq_available(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0) { cudaGetLastError(); return 0; }
    int dev = 0, major = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return 0;
    return major == 10 ? 1 : 0;
}

extern "C" int wf_seq_create(const wf_seq_config* cfg, const wf_seq_layer* layers, wf_seq_engine** out) {
    if (!cfg || !layers || !out) { set_error("wf_seq_create: null argument"); return WF_ERR_INVALID; }
    if (int rc = validate(*cfg, layers)) return rc;
    if (!wf_seq_available()) { set_error("wf_seq_create: no compute-capability-10.x device"); return WF_ERR_UNSUPPORTED; }
    wf_seq_engine* e = new wf_seq_engine();
    e->cfg = *cfg;
    e->dt = cfg->dtype == WF_SEQ_F32 ? WF_F32 : WF_BF16;
    e->esz = e->dt == WF_F32 ? 4 : 2;
    if (const char* pm = getenv("WF_SEQ_PAIR_MAX")) e->pair_path_max = atoi(pm);
    if (const char* am = getenv("WF_SEQ_ATTN_MMA")) e->attn_mma = atoi(am);
    if (const char* gm = getenv("WF_SEQ_GRAPH_MAX")) e->graph_max = atoi(gm);
    if (const char* aw = getenv("WF_SEQ_ATTN_WAVES")) e->attn_waves = atoi(aw) > 0 ? atoi(aw) : 1;
    if (const char* fi = getenv("WF_SEQ_FUSE_INPUT")) e->fuse_input = atoi(fi);
    const wf_seq_config& c = e->cfg;
    const int W = c.width, T = c.max_step_tokens, taps = c.canon_taps;
    int rc = WF_OK;
#define TRY(x) do { if ((rc = (x))) { wf_seq_destroy(e); return rc; } } while (0)
    if (cuda_check(cudaStreamCreateWithFlags(&e->stream, cudaStreamNonBlocking), "stream")) { delete e; return WF_ERR_CUDA; }
    TRY(dalloc_t(e, &e->embed, (size_t)c.vocab * W));
    const bool parallel = c.block_form == WF_SEQ_BLOCK_PARALLEL;
    const bool post = c.block_form == WF_SEQ_BLOCK_POST || parallel;       // both have one norm per sublayer and no input convolution
    const size_t norm_elems = post && !parallel && !c.norm_weights ? 1 : W;   // the post form's norms have a single gain unless the model says otherwise
    TRY(dalloc_t(e, &e->final_norm, norm_elems));
    add_tensor(e, "embed", e->embed, (size_t)c.vocab * W);
    add_tensor(e, "final.norm", e->final_norm, norm_elems);
    if (c.tied_head) e->head = e->embed;
    else { TRY(dalloc_t(e, &e->head, (size_t)c.vocab * W)); add_tensor(e, "head", e->head, (size_t)c.vocab * W); }
    // maxima over layers for the shared workspaces
    size_t max_np = 1, max_hd = 1, max_hr = 1, max_hrot = 1, max_hv = 1, max_C = 1, max_H = 1, max_N = 1, max_top = 1, max_E = 1, max_ff = 1, max_uff = 0, max_gqa_dv = 0;
    long long cache_elems = 0;
    size_t st = 0;
    e->layers.resize(c.n_layers + c.n_extra);
    size_t max_gate = 1, max_decay = 1, max_gfull = 0, max_afull = 0, max_scan = 0, max_qfull = 0, max_qrank = 0;
    bool any_mlstm = false;
    bool own = true;                 // false while a tied layer is laid out: it allocates and names nothing, its weights are its source's
    auto walloc = [&](void** ptr, size_t count) -> int { return own ? dalloc_t(e, ptr, count) : WF_OK; };
    auto name = [&](const std::string& n, void* dst, size_t count) { if (own) add_tensor(e, n, dst, count); };
    // one mixer: weights named mp + '<tensor>', its part of a cache page, its part of a state slot
    auto setup_mixer = [&](LayerState& L, const std::string& mp) -> int {
        const wf_seq_layer& l = L.c;
        int rc = WF_OK;
#define TRYL(x) do { if ((rc = (x))) return rc; } while (0)
        const size_t nv = (size_t)l.heads * l.vdim;
        TRYL(walloc(&L.wo, (size_t)W * nv)); name(mp + "o", L.wo, (size_t)W * nv);
        if (l.type == WF_SEQ_GQA_ATTENTION) {
            const size_t nq = (size_t)l.heads * l.dim, nk = (size_t)l.kv_heads * l.dim, nvk = (size_t)l.kv_heads * l.vdim;
            const bool ownkv = l.kv_from < 0;
            const size_t ng = l.head_gate == 2 ? nv : (size_t)l.heads;
            size_t off = nq;
            const bool ownv = ownkv && !l.v_is_k;       // values that are the keys are neither projected nor cached
            if (ownkv) { L.k_off = (int)off; off += nk; }
            if (ownv) { L.v_off = (int)off; off += nvk; }
            if (l.head_gate) { L.g_off = (int)off; off += ng; }
            L.np = (int)off;
            TRYL(walloc(&L.wp, (size_t)L.np * W));
            name(mp + "q", L.wp, nq * W);
            if (ownkv) {
                name(mp + "k", at(e, L.wp, (size_t)L.k_off * W), nk * W);
                if (ownv) name(mp + "v", at(e, L.wp, (size_t)L.v_off * W), nvk * W);
            }
            if (l.head_gate) name(mp + "g", at(e, L.wp, (size_t)L.g_off * W), ng * W);
            if (l.proj_bias) {
                TRYL(walloc(&L.qb, nq)); name(mp + "q.b", L.qb, nq);
                if (ownkv) {
                    TRYL(walloc(&L.kb, nk)); name(mp + "k.b", L.kb, nk);
                    if (ownv) { TRYL(walloc(&L.vb, nvk)); name(mp + "v.b", L.vb, nvk); }
                }
                if (l.proj_bias == 1) { TRYL(walloc(&L.ob, W)); name(mp + "o.b", L.ob, W); }
            }
            if (l.qk_norm >= WF_SEQ_QKNORM_HEAD) {
                const size_t wq = l.qk_norm == WF_SEQ_QKNORM_FULL ? nq : (size_t)l.dim, wk = l.qk_norm == WF_SEQ_QKNORM_FULL ? nk : (size_t)l.dim;
                TRYL(walloc(&L.q_norm_w, wq)); name(mp + "q.norm", L.q_norm_w, wq);
                TRYL(walloc(&L.k_norm_w, wk)); name(mp + "k.norm", L.k_norm_w, wk);      // a layer that reads another's cache still names it: unused
            }
            if (l.rel_rows > 0) {
                TRYL(walloc(&L.rel, (size_t)l.rel_rows * l.heads)); name(mp + "rel", L.rel, (size_t)l.rel_rows * l.heads);
                // beyond rel_far every distance falls into the last row: rel_far + 1 rows by distance are all there is
                L.rel_n = (int)ceilf(l.rel_far) + 1;
                if (own) TRYL(dalloc_n(e, &L.rel_dist, (size_t)L.rel_n * l.heads));
            }
            if (ownkv) {
                // every layer's part of a page starts 16-byte aligned
                cache_elems = (cache_elems + 7) / 8 * 8;
                L.cache_off = cache_elems;
                cache_elems += (long long)c.page_size * (nk + (ownv ? nvk : 0));
            }
            max_hd = std::max(max_hd, nq); max_gqa_dv = std::max(max_gqa_dv, (size_t)l.vdim);
            max_gate = std::max(max_gate, ng);
        } else if (l.type == WF_SEQ_LATENT_ATTENTION) {
            // fused projection [queries, or their latent | latent and rotated key part | gate logits]
            const size_t nq = (size_t)l.heads * (l.dim + l.rot_dim), nkv = l.kv_rank + l.rot_dim, qcols = l.q_rank > 0 ? (size_t)l.q_rank : nq;
            L.kv_col = (int)qcols;
            L.np = (int)(qcols + nkv + (l.head_gate ? nv : 0));
            TRYL(walloc(&L.wp, (size_t)L.np * W));
            if (l.q_rank > 0) {
                name(mp + "dq", L.wp, qcols * W);
                TRYL(walloc(&L.dq_norm, qcols)); name(mp + "dq.norm", L.dq_norm, qcols);
                TRYL(walloc(&L.uq, nq * qcols)); name(mp + "uq", L.uq, nq * qcols);
                max_qfull = std::max(max_qfull, nq); max_qrank = std::max(max_qrank, qcols);
            } else name(mp + "q", L.wp, nq * W);
            name(mp + "dkv", at(e, L.wp, qcols * W), nkv * W);
            if (l.head_gate) name(mp + "g", at(e, L.wp, (qcols + nkv) * W), nv * W);
            if (l.sink == 2) {
                TRYL(walloc(&L.sink_raw, l.heads)); name(mp + "sink", L.sink_raw, l.heads);
                if (own) TRYL(dalloc_n(e, &L.sink_f, l.heads));
            }
            if (own && l.rope_dims > 0) TRYL(dalloc_n(e, &L.freq, l.rope_dims / 2));
            TRYL(walloc(&L.dkv_norm, l.kv_rank)); name(mp + "dkv.norm", L.dkv_norm, l.kv_rank);
            TRYL(walloc(&L.uk, (size_t)l.heads * l.dim * l.kv_rank)); name(mp + "uk", L.uk, (size_t)l.heads * l.dim * l.kv_rank);
            TRYL(walloc(&L.ukT, (size_t)l.heads * l.dim * l.kv_rank));
            TRYL(walloc(&L.uv, nv * l.kv_rank)); name(mp + "uv", L.uv, nv * l.kv_rank);
            L.cache_off = cache_elems;
            cache_elems += (long long)c.page_size * nkv;
            max_hd = std::max(max_hd, (size_t)l.heads * l.dim); max_hr = std::max(max_hr, (size_t)l.heads * l.kv_rank);
            max_hrot = std::max(max_hrot, (size_t)l.heads * std::max(l.rot_dim, 1));
        } else if (l.type == WF_SEQ_MINGRU) {
            // [z | x | g], all of the channel count; state: one float per channel
            const size_t C = nv;
            L.np = (int)(3 * C);
            TRYL(walloc(&L.wp, (size_t)L.np * W));
            name(mp + "z", L.wp, C * W);
            name(mp + "x", at(e, L.wp, C * W), C * W);
            name(mp + "g", at(e, L.wp, 2 * C * W), C * W);
            TRYL(walloc(&L.gb1, C)); name(mp + "z.b", L.gb1, C);
            TRYL(walloc(&L.gb2, C)); name(mp + "x.b", L.gb2, C);
            L.st_S = st; st += C;
        } else if (l.type == WF_SEQ_MLSTM) {
            // [q | k | v | g | i | f]; state: the matrix with the normaliser as its last column, then the running maximum per head
            const size_t nk = (size_t)l.heads * l.dim;
            L.np = (int)(2 * nk + 2 * nv + 2 * l.heads);
            TRYL(walloc(&L.wp, (size_t)L.np * W));
            name(mp + "q", L.wp, nk * W);
            name(mp + "k", at(e, L.wp, nk * W), nk * W);
            name(mp + "v", at(e, L.wp, 2 * nk * W), nv * W);
            name(mp + "g", at(e, L.wp, (2 * nk + nv) * W), nv * W);
            name(mp + "i", at(e, L.wp, (2 * nk + 2 * nv) * W), (size_t)l.heads * W);
            name(mp + "f", at(e, L.wp, (2 * nk + 2 * nv + l.heads) * W), (size_t)l.heads * W);
            TRYL(walloc(&L.gb1, l.heads)); name(mp + "i.b", L.gb1, l.heads);
            TRYL(walloc(&L.gb2, l.heads)); name(mp + "f.b", L.gb2, l.heads);
            TRYL(walloc(&L.onorm, nv)); name(mp + "norm", L.onorm, nv);
            L.st_S = st; st += (size_t)l.heads * l.dim * (l.vdim + 1);
            L.st_m = st; st += l.heads;
            max_scan = std::max(max_scan, (size_t)l.heads * l.dim * (l.vdim + 1));
            max_hv = std::max(max_hv, (size_t)l.heads * (l.vdim + 1));
            any_mlstm = true;
        } else if (l.type == WF_SEQ_SSD) {
            // [z | x | B | C | dt]: x, B and C are the convolved channels
            const size_t GN = (size_t)l.kv_heads * l.dim;
            L.C = (int)(nv + 2 * GN);
            L.np = (int)(2 * nv + 2 * GN + l.heads);
            TRYL(walloc(&L.wp, (size_t)L.np * W)); name(mp + "in", L.wp, (size_t)L.np * W);
            TRYL(walloc(&L.conv_w, (size_t)L.C * l.conv)); name(mp + "conv", L.conv_w, (size_t)L.C * l.conv);
            TRYL(walloc(&L.conv_b, L.C)); name(mp + "conv.b", L.conv_b, L.C);
            TRYL(walloc(&L.dt_bias, l.heads)); name(mp + "dt_bias", L.dt_bias, l.heads);
            TRYL(walloc(&L.A_log, l.heads)); name(mp + "A_log", L.A_log, l.heads);
            TRYL(walloc(&L.Dskip, l.heads)); name(mp + "D", L.Dskip, l.heads);
            TRYL(walloc(&L.onorm, nv)); name(mp + "norm", L.onorm, nv);
            L.st_conv = st; st += (size_t)(l.conv - 1) * L.C;
            L.st_S = st; st += (size_t)l.heads * l.dim * l.vdim;
            max_C = std::max(max_C, (size_t)L.C);
            max_scan = std::max(max_scan, (size_t)l.heads * l.dim * l.vdim);
        } else {
            // [q | k | v | gate (or its first factor) | write strength | decay (or its first factor)]
            const size_t nqk = (size_t)l.kv_heads * l.dim;
            L.C = (int)(2 * nqk + nv);
            L.n_decay = l.decay_channels ? l.heads * l.dim : l.heads;
            const size_t g_rows = l.gate_rank > 0 ? (size_t)l.gate_rank : nv, a_rows = l.decay_rank > 0 ? (size_t)l.decay_rank : (size_t)L.n_decay;
            L.g_col = L.C; L.b_col = (int)(L.C + g_rows); L.a_col = L.b_col + l.heads;
            L.np = (int)(L.a_col + a_rows);
            TRYL(walloc(&L.wp, (size_t)L.np * W));
            name(mp + "q", L.wp, nqk * W);
            name(mp + "k", at(e, L.wp, nqk * W), nqk * W);
            name(mp + "v", at(e, L.wp, 2 * nqk * W), nv * W);
            name(mp + (l.gate_rank > 0 ? "g1" : "g"), at(e, L.wp, (size_t)L.g_col * W), g_rows * W);
            name(mp + "b", at(e, L.wp, (size_t)L.b_col * W), (size_t)l.heads * W);
            name(mp + (l.decay_rank > 0 ? "a1" : "a"), at(e, L.wp, (size_t)L.a_col * W), a_rows * W);
            if (l.gate_rank > 0) { TRYL(walloc(&L.g2, nv * l.gate_rank)); name(mp + "g2", L.g2, nv * l.gate_rank); max_gfull = std::max(max_gfull, nv); }
            if (l.decay_rank > 0) { TRYL(walloc(&L.a2, (size_t)L.n_decay * l.decay_rank)); name(mp + "a2", L.a2, (size_t)L.n_decay * l.decay_rank); max_afull = std::max(max_afull, (size_t)L.n_decay); }
            TRYL(walloc(&L.conv_w, (size_t)L.C * l.conv));
            name(mp + "q.conv", L.conv_w, nqk * l.conv);
            name(mp + "k.conv", at(e, L.conv_w, nqk * l.conv), nqk * l.conv);
            name(mp + "v.conv", at(e, L.conv_w, 2 * nqk * l.conv), nv * l.conv);
            TRYL(walloc(&L.A_log, l.heads)); name(mp + "A_log", L.A_log, l.heads);
            TRYL(walloc(&L.dt_bias, L.n_decay)); name(mp + "dt_bias", L.dt_bias, L.n_decay);
            TRYL(walloc(&L.onorm, l.vdim)); name(mp + "norm", L.onorm, l.vdim);
            L.st_conv = st; st += (size_t)(l.conv - 1) * L.C;
            L.st_S = st; st += (size_t)l.heads * l.dim * l.vdim;
            max_C = std::max(max_C, (size_t)L.C);
            max_decay = std::max(max_decay, (size_t)L.n_decay);
        }
        max_np = std::max(max_np, (size_t)L.np); max_hv = std::max(max_hv, nv); max_H = std::max(max_H, (size_t)l.heads);
#undef TRYL
        return WF_OK;
    };
    const size_t lnorm = post ? norm_elems : (size_t)W;
    // layers with weights of their own first, then the tied ones (a tie may point forward); the order only decides where a layer's part
    // of a page and of a state slot lies
    std::vector<int> order;
    for (int li = 0; li < c.n_layers; ++li) if (!layers[li].tied) order.push_back(li);
    for (int li = 0; li < c.n_layers; ++li) if (layers[li].tied) order.push_back(li);
    for (int li : order) {
        LayerState& L = e->layers[li];
        own = !layers[li].tied;
        if (!own) L = e->layers[layers[li].tied_to];      // the source's weight pointers; offsets of cache and state are assigned anew below
        L.c = layers[li];
        const wf_seq_layer& l = L.c;
        const std::string p = "l" + std::to_string(li) + ".";
        if (own) L.norm1 = L.norm2 = L.norm1b = L.norm2b = L.canon1 = L.canon2 = nullptr;
        if (post) {
            TRY(walloc(&L.norm1, lnorm)); name(p + "norm1", L.norm1, lnorm);
            if (l.has_ff) { TRY(walloc(&L.norm2, lnorm)); name(p + "norm2", L.norm2, lnorm); }
        } else {
            void** norms[4] = {&L.norm1, &L.norm1b, &L.norm2, &L.norm2b};
            const char* norm_names[4] = {"norm1", "norm1b", "norm2", "norm2b"};
            for (int k = 0; k < (l.has_ff ? 4 : 2); ++k) { TRY(walloc(norms[k], W)); name(p + norm_names[k], *norms[k], W); }
            TRY(walloc(&L.canon1, (size_t)W * taps)); name(p + "canon1", L.canon1, (size_t)W * taps);
            L.st_canon1 = st; st += (size_t)(taps - 1) * W;
            if (l.has_ff) {
                TRY(walloc(&L.canon2, (size_t)W * taps)); name(p + "canon2", L.canon2, (size_t)W * taps);
                L.st_canon2 = st; st += (size_t)(taps - 1) * W;
            }
        }
        TRY(setup_mixer(L, l.pair ? p + "mix.left." : p + "mix."));
        if (l.pair) {
            LayerState& R = e->layers[l.pair];
            if (!own) R = e->layers[e->layers[l.tied_to].pair_state];
            R.c = layers[l.pair];
            L.pair_state = l.pair;
            TRY(setup_mixer(R, p + "mix.right."));
        }
        if (l.has_ff == WF_SEQ_FF_DENSE) {
            L.uff = l.ff; L.ulimit = l.ff_limit;
            const bool gated = l.ff_act != WF_SEQ_ACT_RELU2;
            TRY(walloc(&L.ugu, (size_t)(gated ? 2 : 1) * l.ff * W)); TRY(walloc(&L.ud, (size_t)W * l.ff));
            if (gated) name(p + "mlp.gate", L.ugu, (size_t)l.ff * W);
            name(p + "mlp.up", at(e, L.ugu, gated ? (size_t)l.ff * W : 0), (size_t)l.ff * W);
            name(p + "mlp.down", L.ud, (size_t)W * l.ff);
            max_uff = std::max(max_uff, (size_t)l.ff);
        } else if (l.has_ff == WF_SEQ_FF_ROUTED) {
            const size_t N = l.experts + l.identity;
            L.nz = (int)N + (l.shared_ff > 0 ? 1 : 0);
            TRY(walloc(&L.router, (size_t)L.nz * W)); name(p + "mlp.router", L.router, N * W);
            if (l.shared_ff > 0) {
                L.uff = l.shared_ff; L.ulimit = l.shared_limit;
                name(p + "mlp.shared.sg", at(e, L.router, N * W), W);
                TRY(walloc(&L.ugu, (size_t)2 * l.shared_ff * W)); TRY(walloc(&L.ud, (size_t)W * l.shared_ff));
                name(p + "mlp.shared.gate", L.ugu, (size_t)l.shared_ff * W);
                name(p + "mlp.shared.up", at(e, L.ugu, (size_t)l.shared_ff * W), (size_t)l.shared_ff * W);
                name(p + "mlp.shared.down", L.ud, (size_t)W * l.shared_ff);
                max_uff = std::max(max_uff, (size_t)l.shared_ff);
            }
            TRY(walloc(&L.correction, N)); name(p + "mlp.correction", L.correction, N);
            if (l.experts > 0) {
                TRY(walloc(&L.wgu, (size_t)l.experts * 2 * l.ff * W));
                TRY(walloc(&L.wd, (size_t)l.experts * W * l.ff));
                for (int x = 0; x < l.experts; ++x) {
                    const std::string ep = p + "mlp.e" + std::to_string(x) + ".";
                    name(ep + "gate", at(e, L.wgu, (size_t)x * 2 * l.ff * W), (size_t)l.ff * W);
                    name(ep + "up", at(e, L.wgu, ((size_t)x * 2 + 1) * l.ff * W), (size_t)l.ff * W);
                    name(ep + "down", at(e, L.wd, (size_t)x * W * l.ff), (size_t)W * l.ff);
                }
            }
            max_N = std::max(max_N, (size_t)L.nz); max_top = std::max(max_top, (size_t)l.top); max_E = std::max(max_E, (size_t)std::max(l.experts, 1));
            max_ff = std::max(max_ff, (size_t)std::max(l.ff, 1));
            const int P = (T * l.top + GEMM_BM - 1) / GEMM_BM * GEMM_BM + l.experts * GEMM_BM;
            e->P = std::max(e->P, P);
        }
    }
    own = true;
    // cache pool and state slots
    e->page_stride = cache_elems;
    TRY(dalloc_t(e, &e->pool, (size_t)std::max<long long>(cache_elems, 1) * c.max_pages));
    e->slot_stride = st ? st : 1;
    TRY(dalloc_n(e, &e->state, e->slot_stride * c.slots));
    const int max_blocks = c.max_pages;        // one sequence may hold the whole pool
    e->pt.init(c.max_pages, c.page_size, c.slots, max_blocks);
    e->h_len.assign(c.slots, 0);
    TRY(dalloc_n(e, &e->d_block_table, (size_t)c.slots * max_blocks));
    e->meta_ints = (size_t)4 * T + (size_t)4 * c.slots;
    TRY(dalloc_n(e, &e->d_meta, e->meta_ints));
    if (cuda_check(cudaMallocHost((void**)&e->h_meta, e->meta_ints * 4), "pinned metadata")) { wf_seq_destroy(e); return WF_ERR_CUDA; }
    // workspaces
    TRY(dalloc_n(e, &e->row_inv, (size_t)T * c.norm_groups));
    TRY(dalloc_n(e, &e->x, (size_t)T * W)); TRY(dalloc_n(e, &e->hn, (size_t)T * W)); TRY(dalloc_n(e, &e->y, (size_t)T * W));
    TRY(dalloc_t(e, &e->h_t, (size_t)T * W)); TRY(dalloc_t(e, &e->xn, (size_t)T * W));
    TRY(dalloc_n(e, &e->proj, (size_t)T * max_np));
    TRY(dalloc_t(e, &e->qn, (size_t)T * max_hd)); TRY(dalloc_n(e, &e->qr, (size_t)T * max_hrot)); TRY(dalloc_n(e, &e->qa, (size_t)T * max_hr));
    TRY(dalloc_t(e, &e->olat, (size_t)T * max_hr)); TRY(dalloc_n(e, &e->ov, (size_t)T * max_hv)); TRY(dalloc_t(e, &e->og, (size_t)T * max_hv));
    e->attn_ws_rows = 4 * 148;
    if (e->dt == WF_BF16 && max_hr > 1) TRY(dalloc_bytes(e, (void**)&e->attn_ws, (size_t)e->attn_ws_rows * (max_hr + 2 * max_H) * sizeof(float)));
    TRY(dalloc_n(e, &e->gate, (size_t)T * std::max(max_H, max_gate)));
    if (c.n_extra > 0) TRY(dalloc_n(e, &e->y2, (size_t)T * W));
    if (parallel) TRY(dalloc_t(e, &e->h_t2, (size_t)T * W));
    if (max_qfull) { TRY(dalloc_n(e, &e->qfull, (size_t)T * max_qfull)); TRY(dalloc_t(e, &e->cq, (size_t)T * max_qrank)); }
    if (any_mlstm) TRY(dalloc_n(e, &e->mrun, (size_t)T * max_H));
    if (max_scan && T >= 2 * SCAN_CHUNK) {
        e->scan.chunks = scan_chunks_needed(T, c.slots);
        TRY(dalloc_n(e, &e->scan.local, (size_t)e->scan.chunks * max_scan)); TRY(dalloc_n(e, &e->scan.start, (size_t)e->scan.chunks * max_scan));
        TRY(dalloc_n(e, &e->scan.prod, (size_t)e->scan.chunks * max_H));
    }
    if (max_gfull) TRY(dalloc_n(e, &e->gfull, (size_t)T * max_gfull));
    if (max_afull) TRY(dalloc_n(e, &e->afull, (size_t)T * max_afull));
    if (e->dt == WF_BF16 && max_gqa_dv) { e->gqa_ws_rows = 32768; TRY(dalloc_bytes(e, (void**)&e->gqa_ws, gqa_attn_mma_workspace(e->gqa_ws_rows, 1, (int)max_gqa_dv))); }
    if (max_uff) { TRY(dalloc_n(e, &e->ugu, (size_t)T * 2 * max_uff)); TRY(dalloc_t(e, &e->uhmid, (size_t)T * max_uff)); TRY(dalloc_n(e, &e->uy, (size_t)T * W)); }
    TRY(dalloc_n(e, &e->qkvc, (size_t)T * max_C)); TRY(dalloc_n(e, &e->beta, (size_t)T * max_H)); TRY(dalloc_n(e, &e->decay, (size_t)T * std::max(max_H, max_decay)));
    TRY(dalloc_n(e, &e->od, (size_t)T * max_hv));
    TRY(dalloc_n(e, &e->z, (size_t)T * max_N)); TRY(dalloc_n(e, &e->ids, (size_t)T * max_top)); TRY(dalloc_n(e, &e->wts, (size_t)T * max_top));
    TRY(dalloc_n(e, &e->pair_row, (size_t)T * max_top)); TRY(dalloc_n(e, &e->counts, max_E)); TRY(dalloc_n(e, &e->plan_scratch, 2 * max_E + 1));
    const size_t P = e->P ? e->P : GEMM_BM;
    TRY(dalloc_n(e, &e->sorted_rows, P)); TRY(dalloc_n(e, &e->tile_group, P / GEMM_BM));
    TRY(dalloc_t(e, &e->hperm, P * W));
    TRY(dalloc_n(e, &e->gu, P * 2 * max_ff)); TRY(dalloc_t(e, &e->hmid, P * max_ff)); TRY(dalloc_n(e, &e->yexp, P * W));
#undef TRY
    if (cuda_check(cudaMemsetAsync(e->state, 0, e->slot_stride * c.slots * 4, e->stream), "state")) { wf_seq_destroy(e); return WF_ERR_CUDA; }
    if (cuda_check(cudaMemsetAsync(e->pool, 0, (size_t)std::max<long long>(cache_elems, 1) * c.max_pages * e->esz, e->stream), "pool")) { wf_seq_destroy(e); return WF_ERR_CUDA; }
    if (cuda_check(cudaStreamSynchronize(e->stream), "sync")) { wf_seq_destroy(e); return WF_ERR_CUDA; }
    *out = e;
    return WF_OK;
}

extern "C" void wf_seq_destroy(wf_seq_engine* e) {
    if (!e) return;
    if (e->stream) cudaStreamSynchronize(e->stream);
    for (auto& g : e->graphs) cudaGraphExecDestroy(g.second);
    for (void* p : e->allocs) cudaFree(p);
    if (e->logits) cudaFree(e->logits);
    if (e->d_uniform) cudaFree(e->d_uniform);
    if (e->d_next) cudaFree(e->d_next);
    if (e->h_meta) cudaFreeHost(e->h_meta);
    if (e->stream) cudaStreamDestroy(e->stream);
    delete e;
}

extern "C" size_t wf_seq_device_bytes(const wf_seq_engine* e) { return e ? e->dev_bytes : 0; }
extern "C" int wf_seq_tensor_count(const wf_seq_engine* e) { return e ? (int)e->tensors.size() : 0; }
extern "C" const char* wf_seq_tensor_name(const wf_seq_engine* e, int i, size_t* count, int* loaded) {
    if (!e || i < 0 || i >= (int)e->tensors.size()) return nullptr;
    if (count) *count = e->tensors[i].count;
    if (loaded) *loaded = e->tensors[i].loaded ? 1 : 0;
    return e->tensors[i].name.c_str();
}

extern "C" int wf_seq_set_tensor(wf_seq_engine* e, const char* name, const void* data, size_t count, int is_host) {
    if (!e || !name || !data) { set_error("wf_seq_set_tensor: null argument"); return WF_ERR_INVALID; }
    auto it = e->tensor_index.find(name);
    if (it == e->tensor_index.end()) { set_error("wf_seq_set_tensor: this model has no tensor '%s'", name); return WF_ERR_INVALID; }
    TensorSlot& t = e->tensors[it->second];
    if (count != t.count) { set_error("wf_seq_set_tensor: '%s' holds %zu elements, expected %zu", name, count, t.count); return WF_ERR_INVALID; }
    if (cuda_check(cudaMemcpyAsync(t.dst, data, count * e->esz, is_host ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToDevice, e->stream), "tensor upload")) return WF_ERR_CUDA;
    if (cuda_check(cudaStreamSynchronize(e->stream), "sync")) return WF_ERR_CUDA;
    t.loaded = true;
    e->finalized = false;
    return WF_OK;
}

extern "C" int wf_seq_finalize(wf_seq_engine* e) {
    if (!e) return WF_ERR_INVALID;
    for (const TensorSlot& t : e->tensors)
        if (!t.loaded) { set_error("wf_seq_finalize: tensor '%s' was not loaded", t.name.c_str()); return WF_ERR_INVALID; }
    for (LayerState& L : e->layers)
        if (L.c.type == WF_SEQ_LATENT_ATTENTION)      // W_uk per head [dim, kv_rank] -> [kv_rank, dim]: the weight of q -> W_uk^T q
            if (int rc = launch_transpose_heads(e->dt, L.uk, L.c.heads, L.c.dim, L.c.kv_rank, L.ukT, e->stream)) return rc;
    // attention bias tables: the loaded rows [rel_rows, heads] expanded to one row per distance 0 .. rel_far (later distances share the last).
    // The bucket of a distance is computed here, once, in double: exact below rel_rows / 2, then logarithmic steps up to rel_far.
    for (int li = 0; li < (int)e->layers.size(); ++li) {
        LayerState& L = e->layers[li];
        if (L.c.type != WF_SEQ_GQA_ATTENTION || L.c.rel_rows <= 0 || L.c.tied) continue;     // a tied layer points at its source's table
        const int B = L.c.rel_rows, H = L.c.heads, half = B / 2;
        std::vector<unsigned char> raw((size_t)B * H * e->esz);
        if (cuda_check(cudaMemcpyAsync(raw.data(), L.rel, raw.size(), cudaMemcpyDeviceToHost, e->stream), "bias table D2H")) return WF_ERR_CUDA;
        if (cuda_check(cudaStreamSynchronize(e->stream), "sync")) return WF_ERR_CUDA;
        std::vector<float> tab((size_t)L.rel_n * H);
        for (int n = 0; n < L.rel_n; ++n) {
            int bucket = n;
            if (n >= half) {
                const double steps = floor(log((double)n / (double)half) / log((double)L.c.rel_far / (double)half) * (double)(B - half));
                bucket = steps >= (double)(B - 1 - half) ? B - 1 : half + (int)steps;
            }
            for (int h = 0; h < H; ++h) {
                float v;
                if (e->dt == WF_F32) v = ((const float*)raw.data())[(size_t)bucket * H + h];
                else { const uint32_t bits = (uint32_t)((const uint16_t*)raw.data())[(size_t)bucket * H + h] << 16; memcpy(&v, &bits, 4); }
                tab[(size_t)n * H + h] = v;
            }
        }
        if (cuda_check(cudaMemcpyAsync(L.rel_dist, tab.data(), tab.size() * 4, cudaMemcpyHostToDevice, e->stream), "bias table H2D")) return WF_ERR_CUDA;
        if (cuda_check(cudaStreamSynchronize(e->stream), "sync")) return WF_ERR_CUDA;
    }
    // latent attention: the rotation's frequencies, tabulated in double (with frequency interpolation: pairs whose wavelength is long
    // against the original context turn `factor` times slower, short ones as they are, a linear ramp over the pair index between), and
    // the learned sinks as floats
    for (LayerState& L : e->layers) {
        if (L.c.type != WF_SEQ_LATENT_ATTENTION || L.c.tied) continue;
        const wf_seq_layer& l = L.c;
        if (L.freq) {
            const int dims = l.rope_dims, half = dims / 2;
            const double base = l.rope_base, pi = 3.14159265358979323846;
            std::vector<double> f(half);
            for (int i = 0; i < half; ++i) f[i] = pow(base, -2.0 * i / dims);
            L.rope_mscale = 1.f;
            if (l.rope_factor > 0.f) {
                const double factor = l.rope_factor;
                auto pair_of = [&](double turns) { return dims * log((double)l.rope_orig / (2.0 * pi * turns)) / (2.0 * log(base)); };
                const double lo = std::max(floor(pair_of(l.rope_fast)), 0.0), hi = std::min(ceil(pair_of(l.rope_slow)), (double)(dims - 1));
                for (int i = 0; i < half; ++i) {
                    const double ramp = std::min(std::max(((double)i - lo) / std::max(hi - lo, 0.001), 0.0), 1.0);
                    f[i] = f[i] / factor * ramp + f[i] * (1.0 - ramp);
                }
                L.rope_mscale = (float)(0.1 * log(factor) + 1.0);
            }
            if (cuda_check(cudaMemcpyAsync(L.freq, f.data(), f.size() * sizeof(double), cudaMemcpyHostToDevice, e->stream), "rotation table H2D")) return WF_ERR_CUDA;
            if (cuda_check(cudaStreamSynchronize(e->stream), "sync")) return WF_ERR_CUDA;
        }
        if (L.sink_f) {
            std::vector<unsigned char> raw((size_t)l.heads * e->esz);
            if (cuda_check(cudaMemcpyAsync(raw.data(), L.sink_raw, raw.size(), cudaMemcpyDeviceToHost, e->stream), "sinks D2H")) return WF_ERR_CUDA;
            if (cuda_check(cudaStreamSynchronize(e->stream), "sync")) return WF_ERR_CUDA;
            std::vector<float> sf(l.heads);
            for (int h = 0; h < l.heads; ++h) {
                if (e->dt == WF_F32) sf[h] = ((const float*)raw.data())[h];
                else { const uint32_t bits = (uint32_t)((const uint16_t*)raw.data())[h] << 16; memcpy(&sf[h], &bits, 4); }
            }
            if (cuda_check(cudaMemcpyAsync(L.sink_f, sf.data(), sf.size() * 4, cudaMemcpyHostToDevice, e->stream), "sinks H2D")) return WF_ERR_CUDA;
            if (cuda_check(cudaStreamSynchronize(e->stream), "sync")) return WF_ERR_CUDA;
        }
    }
    // tied latent layers use their source's tables
    for (LayerState& L : e->layers)
        if (L.c.type == WF_SEQ_LATENT_ATTENTION && L.c.tied) { const LayerState& S = e->layers[L.c.tied_to]; L.freq = S.freq; L.sink_f = S.sink_f; L.rope_mscale = S.rope_mscale; }
    if (cuda_check(cudaStreamSynchronize(e->stream), "finalize")) return WF_ERR_CUDA;
    e->finalized = true;
    return WF_OK;
}

extern "C" int wf_seq_admit(wf_seq_engine* e, int* slot) {
    if (!e || !slot) return WF_ERR_INVALID;
    const int s = e->pt.acquire_slot();
    *slot = s;
    if (s < 0) return WF_OK;
    e->h_len[s] = 0;
    // a slot that is used again must not carry the previous sequence's convolution tails or recurrent state
    if (cuda_check(cudaMemsetAsync(e->state + (size_t)s * e->slot_stride, 0, e->slot_stride * 4, e->stream), "state reset")) return WF_ERR_CUDA;
    return WF_OK;
}

extern "C" int wf_seq_release(wf_seq_engine* e, int slot) {
    if (!e || slot < 0 || slot >= e->cfg.slots || !e->pt.live[slot]) { set_error("wf_seq_release: slot %d is not live", slot); return WF_ERR_INVALID; }
    e->pt.release_slot(slot);
    e->h_len[slot] = 0;
    return WF_OK;
}

extern "C" int wf_seq_length(const wf_seq_engine* e, int slot) { return (e && slot >= 0 && slot < e->cfg.slots) ? e->h_len[slot] : -1; }
extern "C" int wf_seq_free_pages(const wf_seq_engine* e) { return e ? (int)e->pt.free_pages.size() : 0; }
extern "C" int wf_seq_free_slots(const wf_seq_engine* e) { return e ? (int)e->pt.free_slots.size() : 0; }
extern "C" void* wf_seq_logits_device(wf_seq_engine* e) { return e ? e->logits : nullptr; }
extern "C" int wf_seq_launches_last_step(const wf_seq_engine* e) { return e ? e->launches : 0; }
extern "C" int wf_seq_set_layer_tap(wf_seq_engine* e, float* host) { if (!e) return WF_ERR_INVALID; e->layer_tap = host; return WF_OK; }

extern "C" int wf_seq_step(wf_seq_engine* e, int nseq, const int32_t* slots, const int32_t* counts, const int32_t* tokens, int nwant,
                           const int32_t* want, float* logits_host) {
    if (!e || !slots || !counts || !tokens || (nwant > 0 && !want)) { set_error("wf_seq_step: null argument"); return WF_ERR_INVALID; }
    StepView v;
    int rc;
    if ((rc = prepare_step(e, nseq, slots, counts, tokens, nwant, want, &v))) return rc;
    const long long l0 = launch_count();
    if ((rc = run_model(e, v, nwant))) return rc;
    if (launch_count() > l0) e->launches = (int)(launch_count() - l0);     // a graph replay launches what its capture counted
    if (logits_host && nwant > 0)
        if (cuda_check(cudaMemcpyAsync(logits_host, e->logits, (size_t)nwant * e->cfg.vocab * 4, cudaMemcpyDeviceToHost, e->stream), "logits D2H")) return WF_ERR_CUDA;
    if (cuda_check(cudaStreamSynchronize(e->stream), "wf_seq_step")) return WF_ERR_CUDA;
    if (e->dt == WF_BF16 && gemm_tc_error(e->stream)) { set_error("wf_seq_step: a bounded wait of the tensor-core matrix product ran out"); return WF_ERR_CUDA; }
    commit_lengths(e, nseq, slots, counts);
    return WF_OK;
}

extern "C" int wf_seq_sample(wf_seq_engine* e, int nwant, float temperature, int top_k, float top_p, const float* uniforms_host, int32_t* next_host) {
    if (!e || !next_host || nwant <= 0 || (size_t)nwant > e->logits_rows) { set_error("wf_seq_sample: no logits for %d rows", nwant); return WF_ERR_INVALID; }
    if ((size_t)nwant > e->sample_rows) {
        if (e->d_uniform) cudaFree(e->d_uniform);
        if (e->d_next) cudaFree(e->d_next);
        e->d_uniform = nullptr; e->d_next = nullptr; e->sample_rows = 0;
        if (cuda_check(cudaMalloc((void**)&e->d_uniform, (size_t)nwant * 4), "cudaMalloc")) return WF_ERR_CUDA;
        if (cuda_check(cudaMalloc((void**)&e->d_next, (size_t)nwant * 4), "cudaMalloc")) return WF_ERR_CUDA;
        e->sample_rows = nwant;
    }
    if (temperature > 0.f) {
        if (!uniforms_host) { set_error("wf_seq_sample: uniforms required when temperature > 0"); return WF_ERR_INVALID; }
        if (cuda_check(cudaMemcpyAsync(e->d_uniform, uniforms_host, (size_t)nwant * 4, cudaMemcpyHostToDevice, e->stream), "uniforms H2D")) return WF_ERR_CUDA;
    }
    if (int rc = launch_sample(e->logits, nwant, e->cfg.vocab, temperature, top_k, top_p, e->d_uniform, e->d_next, e->stream)) return rc;
    if (cuda_check(cudaMemcpyAsync(next_host, e->d_next, (size_t)nwant * 4, cudaMemcpyDeviceToHost, e->stream), "next D2H")) return WF_ERR_CUDA;
    return cuda_check(cudaStreamSynchronize(e->stream), "wf_seq_sample");
}

extern "C" int wf_seq_run_part(wf_seq_engine* e, int layer, int part, int nseq, const int32_t* slots, const int32_t* counts, const float* in_host,
                               float* out_host) {
    if (!e || !slots || !counts || !in_host || !out_host || layer < 0 || layer >= e->cfg.n_layers) { set_error("wf_seq_run_part: bad argument"); return WF_ERR_INVALID; }
    StepView v;
    int rc;
    if ((rc = prepare_step(e, nseq, slots, counts, nullptr, 0, nullptr, &v))) return rc;
    LayerState& L = e->layers[layer];
    const int W = e->cfg.width, n = v.b.n;
    cudaStream_t s = e->stream;
    const size_t bytes = (size_t)n * W * 4;
    float* result = e->y;
    const bool parallel = e->cfg.block_form == WF_SEQ_BLOCK_PARALLEL;
    const bool post = e->cfg.block_form == WF_SEQ_BLOCK_POST || parallel;
    if (part == 5 && !(parallel && L.c.has_ff)) { set_error("wf_seq_run_part: layer %d has no second norm", layer); return WF_ERR_INVALID; }
    if (post && (part == 1 || part == 4)) { set_error("wf_seq_run_part: this model's sublayers have no input convolution"); return WF_ERR_INVALID; }
    if ((part == 0 || part == 5) && parallel) {
        if (cuda_check(cudaMemcpyAsync(e->x, in_host, bytes, cudaMemcpyHostToDevice, s), "in")) return WF_ERR_CUDA;
        rc = launch_group_rmsnorm(e->dt, e->x, W, part == 0 ? L.norm1 : L.norm2, 1, e->cfg.eps, n, W, nullptr, e->hn, W, nullptr, 0, nullptr, s, nullptr, 1.f, 0.f, e->cfg.norm_offset);
        result = e->hn;
    } else if (part == 0 && post && e->cfg.norm_weights) {
        if (cuda_check(cudaMemcpyAsync(e->x, in_host, bytes, cudaMemcpyHostToDevice, s), "in")) return WF_ERR_CUDA;
        rc = launch_group_rmsnorm(e->dt, e->x, W, L.norm1, 1, e->cfg.eps, n, W, nullptr, e->hn, W, nullptr, 0, nullptr, s);
        result = e->hn;
    } else if (part == 0 && post) {
        if (cuda_check(cudaMemcpyAsync(e->x, in_host, bytes, cudaMemcpyHostToDevice, s), "in")) return WF_ERR_CUDA;
        rc = launch_scalar_rmsnorm(e->dt, e->x, W, nullptr, L.norm1, e->cfg.residual_mult, e->cfg.eps, n, W, nullptr, e->hn, W, nullptr, 0, nullptr, s);
        result = e->hn;
    } else if (part == 0) {
        if (cuda_check(cudaMemcpyAsync(e->x, in_host, bytes, cudaMemcpyHostToDevice, s), "in")) return WF_ERR_CUDA;
        rc = launch_group_rmsnorm(e->dt, e->x, W, L.norm1, e->cfg.norm_groups, e->cfg.eps, n, W, nullptr, e->hn, W, nullptr, 0, nullptr, s);
        result = e->hn;
    } else if (part == 1 || part == 4) {
        if (part == 4 && !L.c.has_ff) { set_error("wf_seq_run_part: layer %d has no feed-forward", layer); return WF_ERR_INVALID; }
        if (cuda_check(cudaMemcpyAsync(e->hn, in_host, bytes, cudaMemcpyHostToDevice, s), "in")) return WF_ERR_CUDA;
        const size_t off = part == 1 ? L.st_canon1 : L.st_canon2;
        rc = launch_causal_taps(e->dt, v.b, e->hn, W, part == 1 ? L.canon1 : L.canon2, e->cfg.canon_taps, W, e->state + off, e->slot_stride, 1, 0, nullptr, 0, e->y, W, s);
        if (!rc) rc = launch_taps_state(v.b, e->hn, W, e->cfg.canon_taps, W, e->state + off, e->slot_stride, s);
    } else if (part == 2 || part == 3) {
        if (part == 3 && !L.c.has_ff) { set_error("wf_seq_run_part: layer %d has no feed-forward", layer); return WF_ERR_INVALID; }
        if (cuda_check(cudaMemcpyAsync(e->hn, in_host, bytes, cudaMemcpyHostToDevice, s), "in")) return WF_ERR_CUDA;
        // round the given rows to the storage type exactly as the input convolution's output would be (the post form's sublayers also
        // read the float rows themselves: they are the stream)
        if (post && cuda_check(cudaMemcpyAsync(e->x, e->hn, bytes, cudaMemcpyDeviceToDevice, s), "in")) return WF_ERR_CUDA;
        rc = launch_gate_mul(e->dt, e->hn, W, e->hn, W, 2, n, W, e->h_t, W, s);
        if (!rc) rc = part == 2 ? run_mixer(e, L, v.b) : run_ff(e, L, v.b);
        if (!rc && part == 2 && L.ob && post && !parallel && !e->cfg.norm_weights && !L.c.pair) rc = launch_add_bias(e->dt, e->y, W, L.ob, n, W, s);
    } else { set_error("wf_seq_run_part: unknown part %d", part); return WF_ERR_INVALID; }
    if (rc) return rc;
    if (cuda_check(cudaMemcpyAsync(out_host, result, bytes, cudaMemcpyDeviceToHost, s), "out")) return WF_ERR_CUDA;
    if (cuda_check(cudaStreamSynchronize(s), "wf_seq_run_part")) return WF_ERR_CUDA;
    commit_lengths(e, nseq, slots, counts);
    return WF_OK;
}

extern "C" int wf_seq_time_step(wf_seq_engine* e, int nseq, const int32_t* slots, const int32_t* counts, int iters, float* ms_out);

extern "C" int wf_seq_set_length(wf_seq_engine* e, int slot, int len) {
    if (!e || slot < 0 || slot >= e->cfg.slots || !e->pt.live[slot] || len < 0) { set_error("wf_seq_set_length: bad slot / length"); return WF_ERR_INVALID; }
    e->pt.truncate(slot, len);
    if (!e->pt.ensure(slot, len)) { set_error("wf_seq_set_length: cache pool exhausted"); return WF_ERR_INVALID; }
    e->h_len[slot] = len;
    return WF_OK;
}

extern "C" int wf_seq_profile_step(wf_seq_engine* e, int nseq, const int32_t* slots, const int32_t* counts, int iters, char* out, size_t cap) {
    if (!e || !out || cap < 64) { set_error("wf_seq_profile_step: bad argument"); return WF_ERR_INVALID; }
    e->prof = true;
    e->marks.clear();
    float ms = 0.f;
    mark(e, "start");
    const int rc = wf_seq_time_step(e, nseq, slots, counts, iters, &ms);
    e->prof = false;
    std::map<std::string, std::pair<double, int>> acc;
    if (!rc) {
        // the untimed passes of wf_seq_time_step are included: iters + 2 passes
        for (size_t i = 1; i < e->marks.size(); ++i) {
            float t = 0.f;
            cudaEventElapsedTime(&t, e->marks[i - 1].second, e->marks[i].second);
            auto& a = acc[e->marks[i].first];
            a.first += t; a.second += 1;
        }
    }
    for (auto& m : e->marks) cudaEventDestroy(m.second);
    e->marks.clear();
    if (rc) return rc;
    std::string js = "{";
    char buf[160];
    for (auto& kv : acc) {
        snprintf(buf, sizeof buf, "%s\"%s\": [%.6f, %d]", js.size() > 1 ? ", " : "", kv.first.c_str(), kv.second.first / (iters + 2), kv.second.second / (iters + 2));
        js += buf;
    }
    js += "}";
    if (js.size() + 1 > cap) { set_error("wf_seq_profile_step: output buffer too small"); return WF_ERR_INVALID; }
    memcpy(out, js.c_str(), js.size() + 1);
    return WF_OK;
}

extern "C" int wf_seq_time_step(wf_seq_engine* e, int nseq, const int32_t* slots, const int32_t* counts, int iters, float* ms_out) {
    if (!e || !slots || !counts || !ms_out || iters <= 0) { set_error("wf_seq_time_step: bad argument"); return WF_ERR_INVALID; }
    int n = 0;
    for (int i = 0; i < nseq; ++i) n += counts[i];
    if (n <= 0 || n > e->cfg.max_step_tokens) { set_error("wf_seq_time_step: %d tokens", n); return WF_ERR_INVALID; }
    std::vector<int32_t> tokens(n), want(nseq);
    for (int i = 0; i < n; ++i) tokens[i] = (int32_t)((1103515245u * (unsigned)i + 12345u) % (unsigned)e->cfg.vocab);
    int at_ = 0;
    for (int i = 0; i < nseq; ++i) { at_ += counts[i]; want[i] = at_ - 1; }
    StepView v;
    int rc;
    if ((rc = prepare_step(e, nseq, slots, counts, tokens.data(), nseq, want.data(), &v))) return rc;
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0); cudaEventCreate(&e1);
    for (int it = -2; it < iters; ++it) {      // two untimed passes first (the second one captures the graph of a decode shape)
        if (it == 0) cudaEventRecord(e0, e->stream);
        const long long l0 = launch_count();
        if ((rc = run_model(e, v, nseq))) break;
        if (it == -2) e->launches = (int)(launch_count() - l0);      // the eager pass: what one step launches
    }
    cudaEventRecord(e1, e->stream);
    const cudaError_t ce = cudaStreamSynchronize(e->stream);
    float ms = 0.f;
    if (!rc && ce == cudaSuccess) cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0); cudaEventDestroy(e1);
    for (int i = 0; i < nseq; ++i) e->pt.truncate(slots[i], e->h_len[slots[i]]);   // the timed tokens are not kept
    if (rc) return rc;
    if (cuda_check(ce, "wf_seq_time_step")) return WF_ERR_CUDA;
    *ms_out = ms / iters;
    return WF_OK;
}
