// Host side of a decode step: the reference's ForwardPassPipeline (token embedding -> transformer blocks
// -> language-model head -> sampler, bitnet-inference/src/engine/forward_pass_pipeline.rs:146-362) for ONE
// new token per sequence with a KV cache, every BitLinear on the kernels of this library.
//
//   block (TransformerBlock::forward, transformer_layers.rs:675-709):
//     x += previous block's FFN output; n = SubLN(x)        -- inside the q/k/v quantiser launch
//     q, k, v = BitLinear(n)                                -- one launch, weights stacked
//     a = attention(q, cache + (k, v))                      -- bf16 cache, appended in the same launch
//     o = BitLinear(a)
//     x += o; n = SubLN(x)                                  -- inside the gate/up quantiser launch
//     f = down(up(n) * relu(gate(n))^2)
//   logits = BitLinear_lm_head(x + f)  (no final normalisation, forward_pass_pipeline.rs:283-291)
//   next = sample(logits)
//
// A step is recorded once per batch size as a CUDA graph whose inputs (token ids, positions, generator
// states) live in device memory, so that generating n tokens is n graph launches without a host round trip.
#include <cstring>
#include <mutex>
#include <new>
#include <vector>

#include "common.cuh"

using namespace bitnet;

namespace {

struct DecLayer {
    uint8_t *qkv = nullptr, *o = nullptr, *gate = nullptr, *up = nullptr, *down = nullptr;
    float s_q = 1, s_k = 1, s_v = 1, s_o = 1, s_g = 1, s_u = 1, s_d = 1;
    float *n1w = nullptr, *n1b = nullptr, *n2w = nullptr, *n2b = nullptr;
    bool loaded = false;
};

struct StepGraph {
    int kind;   // 0: context step (no head, no sampler), 1: generation step
    size_t batch;
    bitnet_sampling_config sampling;
    int eos;
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
};

}  // namespace

struct bitnet_decoder {
    bitnet_backend *backend = nullptr;
    bitnet_decoder_config cfg = {};
    int device = 0;
    cudaStream_t stream = nullptr;
    std::vector<void *> owned;   // every device allocation, for destroy
    float *embed = nullptr;
    bool embed_loaded = false, head_loaded = false;
    std::vector<DecLayer> layers;
    uint8_t *lm_head = nullptr;
    float s_lm = 1.0f;
    void *kcache = nullptr, *vcache = nullptr;   // [layer][max_batch][kv_heads][max_seq][head_dim] bf16
    int *ids = nullptr, *pos = nullptr, *next = nullptr, *finished = nullptr, *history = nullptr, *step_counter = nullptr;
    int *feed = nullptr;   // [max_seq][max_batch] context tokens of bitnet_decoder_feed
    unsigned long long *rng = nullptr;
    size_t history_rows = 0;
    float *x = nullptr, *qkv = nullptr, *attn = nullptr, *o_out = nullptr, *h = nullptr, *f = nullptr, *logits = nullptr;
    void *ws = nullptr;
    size_t ws_bytes = 0;
    void *attn_scratch = nullptr;
    size_t attn_scratch_bytes = 0;
    std::vector<StepGraph> graphs;
    std::mutex mu;
    bool rng_seeded = false;
    unsigned long long rng_seed = 0;
    size_t host_positions = 0;   // tokens cached per sequence (all sequences advance together)
    size_t batch_in_use = 0;
    bool use_graphs = true;
};

static bitnet_status_t dec_alloc(bitnet_decoder *d, size_t bytes, void **out)
{
    BITNET_TRY(bitnet_backend_allocate(d->backend, bytes ? bytes : 256, out));
    d->owned.push_back(*out);
    return BITNET_OK;
}

static size_t kv_dim(const bitnet_decoder_config &c) { return c.num_kv_heads * c.head_dim; }
static size_t q_dim(const bitnet_decoder_config &c) { return c.num_heads * c.head_dim; }
static size_t cache_layer_elems(const bitnet_decoder_config &c) { return c.max_batch * c.num_kv_heads * c.max_seq_len * c.head_dim; }

// Queues one step for `B` sequences on the decoder's stream.  kind 0: context step (the token is cached,
// nothing is sampled); kind 1: generation step.
static bitnet_status_t enqueue_step(bitnet_decoder *d, size_t B, int kind, const bitnet_sampling_config &sc, int eos)
{
    const bitnet_decoder_config &c = d->cfg;
    const size_t H = c.hidden_size, QD = q_dim(c), KD = kv_dim(c), F = c.ffn_size;
    cudaStream_t s = d->stream;
    bitnet_forward_opts o = {};
    o.flags = BITNET_FLAG_PDL;
    BITNET_TRY(launch_embed_gather(d->ids, d->embed, d->x, B, H, c.vocab_size, s));
    const int n_splits = attention_splits(B, c.num_kv_heads, c.max_seq_len);
    for (size_t l = 0; l < c.num_layers; ++l) {
        const DecLayer &L = d->layers[l];
        bitnet_stack st = {};
        st.n_members = 3;
        st.rows[0] = QD; st.rows[1] = KD; st.rows[2] = KD;
        st.scales[0] = L.s_q; st.scales[1] = L.s_k; st.scales[2] = L.s_v;
        bitnet_row_glue g1 = {};
        if (l > 0) { g1.residual_dev = d->f; g1.sum_out_dev = d->x; }
        g1.norm_weight_dev = L.n1w; g1.norm_bias_dev = L.n1b; g1.norm_eps = c.norm_eps;
        BITNET_TRY(bitnet_bitlinear_forward_fused(L.qkv, &st, d->x, &g1, d->qkv, B, H, &o, d->ws, d->ws_bytes, s));
        char *kc = static_cast<char *>(d->kcache) + l * cache_layer_elems(c) * 2;
        char *vc = static_cast<char *>(d->vcache) + l * cache_layer_elems(c) * 2;
        BITNET_TRY(launch_attention_decode(d->qkv, QD + 2 * KD, QD, QD + KD, kc, vc, d->pos, d->attn, B, c.num_heads, c.num_kv_heads,
                                           c.head_dim, c.max_seq_len, n_splits, d->attn_scratch, d->attn_scratch_bytes, o.flags, s));
        BITNET_TRY(bitnet_bitlinear_forward(L.o, L.s_o, d->attn, d->o_out, B, QD, H, &o, d->ws, d->ws_bytes, s));
        bitnet_row_glue g2 = {};
        g2.residual_dev = d->o_out; g2.sum_out_dev = d->x;
        g2.norm_weight_dev = L.n2w; g2.norm_bias_dev = L.n2b; g2.norm_eps = c.norm_eps;
        BITNET_TRY(bitnet_ffn_forward_fused(L.gate, L.s_g, L.up, L.s_u, L.down, L.s_d, d->x, &g2, d->h, d->f, B, H, F, &o, d->ws,
                                            d->ws_bytes, s));
    }
    if (kind == 0) return BITNET_OK;   // the token is cached now; nothing to sample (the next id comes from the caller's context)
    bitnet_stack st = {};
    st.n_members = 1;
    st.rows[0] = c.vocab_size;
    st.scales[0] = d->s_lm;
    bitnet_row_glue g = {};
    if (c.num_layers > 0) { g.residual_dev = d->f; g.sum_out_dev = d->x; }
    BITNET_TRY(bitnet_bitlinear_forward_fused(d->lm_head, &st, d->x, c.num_layers > 0 ? &g : nullptr, d->logits, B, H, &o, d->ws,
                                              d->ws_bytes, s));
    return launch_sample(d->logits, B, c.vocab_size, sc, d->rng, d->next, d->ids, d->pos, d->history, d->step_counter, eos,
                         d->finished, o.flags, s);
}

// advances the positions after a context step (the generation step's sampler does it itself)
__global__ void advance_pos_kernel(int *pos, int B)
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < B) pos[i] += 1;
}

static bitnet_status_t enqueue_full_step(bitnet_decoder *d, size_t B, int kind, const bitnet_sampling_config &sc, int eos)
{
    BITNET_TRY(enqueue_step(d, B, kind, sc, eos));
    if (kind == 0) {
        cudaLaunchConfig_t lc = {};
        cudaLaunchAttribute attrs[1];
        lc.gridDim = dim3((unsigned)((B + 127) / 128));
        lc.blockDim = dim3(128);
        lc.stream = d->stream;
        attrs[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attrs[0].val.programmaticStreamSerializationAllowed = 1;
        lc.attrs = attrs;
        lc.numAttrs = 1;
        BITNET_CUDA(cudaLaunchKernelEx(&lc, advance_pos_kernel, d->pos, (int)B));
    }
    return BITNET_OK;
}

static bool same_sampling(const bitnet_sampling_config &a, const bitnet_sampling_config &b)
{
    return a.temperature == b.temperature && a.top_k == b.top_k && a.top_p == b.top_p && a.deterministic == b.deterministic;
}

// Launches one step: a recorded graph when graphs are on (recorded on first use), plain launches otherwise.
static bitnet_status_t run_step(bitnet_decoder *d, size_t B, int kind, const bitnet_sampling_config &sc, int eos)
{
    if (!d->use_graphs) return enqueue_full_step(d, B, kind, sc, eos);
    for (StepGraph &g : d->graphs)
        if (g.kind == kind && g.batch == B && g.eos == eos && (kind == 0 || same_sampling(g.sampling, sc))) {
            BITNET_CUDA(cudaGraphLaunch(g.exec, d->stream));
            return BITNET_OK;
        }
    StepGraph g;
    g.kind = kind; g.batch = B; g.sampling = sc; g.eos = eos;
    BITNET_CUDA(cudaStreamBeginCapture(d->stream, cudaStreamCaptureModeThreadLocal));
    const bitnet_status_t q = enqueue_full_step(d, B, kind, sc, eos);
    const cudaError_t err = cudaStreamEndCapture(d->stream, &g.graph);
    if (q != BITNET_OK) {
        if (g.graph) cudaGraphDestroy(g.graph);
        cudaGetLastError();
        return q;
    }
    BITNET_CUDA(err);
    const cudaError_t ierr = cudaGraphInstantiate(&g.exec, g.graph, 0);
    if (ierr != cudaSuccess) {
        cudaGraphDestroy(g.graph);
        return check_cuda(ierr, "cudaGraphInstantiate");
    }
    d->graphs.push_back(g);
    BITNET_CUDA(cudaGraphLaunch(g.exec, d->stream));
    return BITNET_OK;
}

extern "C" void bitnet_decoder_config_default(bitnet_decoder_config *c)
{
    if (!c) return;
    memset(c, 0, sizeof(*c));
    // TransformerConfig / ForwardPassConfig defaults (transformer_layers.rs:36-49, forward_pass_pipeline.rs:99-118)
    c->vocab_size = 128256;
    c->hidden_size = 2048;
    c->num_layers = 12;
    c->num_heads = 16;
    c->num_kv_heads = 16;
    c->head_dim = 128;
    c->ffn_size = 5632;
    c->max_seq_len = 2048;
    c->max_batch = 1;
    c->norm_eps = 1e-5f;
}

extern "C" void bitnet_sampling_config_default(bitnet_sampling_config *c)
{
    if (!c) return;
    c->temperature = 1.0f;   // SamplingConfig::default, sampling.rs:32-45
    c->top_k = 0;
    c->top_p = 1.0f;
    c->seed = 0;
    c->deterministic = 0;
}

extern "C" void bitnet_decoder_destroy(bitnet_decoder *d)
{
    if (!d) return;
    cudaSetDevice(d->device);
    if (d->stream) cudaStreamSynchronize(d->stream);
    for (StepGraph &g : d->graphs) {
        if (g.exec) cudaGraphExecDestroy(g.exec);
        if (g.graph) cudaGraphDestroy(g.graph);
    }
    for (void *p : d->owned) bitnet_backend_free(d->backend, p);
    if (d->stream) cudaStreamDestroy(d->stream);
    delete d;
}

extern "C" bitnet_status_t bitnet_decoder_create(bitnet_backend *b, const bitnet_decoder_config *cfg, bitnet_decoder **out)
{
    if (!b || !cfg || !out) return fail(BITNET_ERR_NULL_POINTER, "bitnet_decoder_create: null argument");
    *out = nullptr;
    const bitnet_decoder_config c = *cfg;
    if (!c.vocab_size || !c.hidden_size || !c.num_heads || !c.num_kv_heads || !c.head_dim || !c.ffn_size || !c.max_seq_len || !c.max_batch)
        return fail(BITNET_ERR_INVALID_CONFIG, "decoder: every size must be positive");
    if (c.num_heads % c.num_kv_heads) return fail(BITNET_ERR_INVALID_CONFIG, "decoder: heads must be a multiple of KV heads");
    if (c.hidden_size % 64 || c.ffn_size % 64 || (c.num_heads * c.head_dim) % 64 || c.hidden_size > 16384 || c.ffn_size > 16384)
        return fail(BITNET_ERR_INVALID_CONFIG, "decoder: hidden, ffn and heads x head_dim must be multiples of 64, at most 16384");
    if (c.head_dim != 64 && c.head_dim != 128) return fail(BITNET_ERR_INVALID_CONFIG, "decoder: head_dim must be 64 or 128");
    const size_t G = c.num_heads / c.num_kv_heads;
    if (G != 1 && G != 2 && G != 4 && G != 8) return fail(BITNET_ERR_INVALID_CONFIG, "decoder: 1, 2, 4 or 8 query heads per KV head");
    bitnet_stream_t s0 = nullptr;
    BITNET_TRY(bitnet_backend_stream(b, 0, &s0));   // also validates the backend

    bitnet_decoder *d = new (std::nothrow) bitnet_decoder();
    if (!d) return fail(BITNET_ERR_MEMORY_ALLOCATION, "out of host memory");
    d->backend = b;
    d->cfg = c;
    d->layers.resize(c.num_layers);
    BITNET_CUDA(cudaGetDevice(&d->device));
    bitnet_status_t st = check_cuda(cudaStreamCreateWithFlags(&d->stream, cudaStreamNonBlocking), "cudaStreamCreateWithFlags");
    const size_t H = c.hidden_size, QD = q_dim(c), KD = kv_dim(c), F = c.ffn_size, B = c.max_batch, V = c.vocab_size;
    auto A = [&](size_t bytes, void **p) { if (st == BITNET_OK) st = dec_alloc(d, bytes, p); };
    A(V * H * 4, reinterpret_cast<void **>(&d->embed));
    A((V * H + 3) / 4 + 256, reinterpret_cast<void **>(&d->lm_head));
    for (size_t l = 0; l < c.num_layers; ++l) {
        DecLayer &L = d->layers[l];
        A((QD + 2 * KD) * H / 4, reinterpret_cast<void **>(&L.qkv));
        A(H * QD / 4, reinterpret_cast<void **>(&L.o));
        A(F * H / 4, reinterpret_cast<void **>(&L.gate));
        A(F * H / 4, reinterpret_cast<void **>(&L.up));
        A(H * F / 4, reinterpret_cast<void **>(&L.down));
        A(H * 4, reinterpret_cast<void **>(&L.n1w)); A(H * 4, reinterpret_cast<void **>(&L.n1b));
        A(H * 4, reinterpret_cast<void **>(&L.n2w)); A(H * 4, reinterpret_cast<void **>(&L.n2b));
    }
    A(c.num_layers * cache_layer_elems(c) * 2, &d->kcache);
    A(c.num_layers * cache_layer_elems(c) * 2, &d->vcache);
    A(B * 4, reinterpret_cast<void **>(&d->ids)); A(B * 4, reinterpret_cast<void **>(&d->pos));
    A(B * 4, reinterpret_cast<void **>(&d->next)); A(B * 4, reinterpret_cast<void **>(&d->finished));
    A(256, reinterpret_cast<void **>(&d->step_counter));
    A(B * 8, reinterpret_cast<void **>(&d->rng));
    d->history_rows = c.max_seq_len;
    A(d->history_rows * B * 4, reinterpret_cast<void **>(&d->history));
    A(c.max_seq_len * B * 4, reinterpret_cast<void **>(&d->feed));
    A(B * H * 4, reinterpret_cast<void **>(&d->x));
    A(B * (QD + 2 * KD) * 4, reinterpret_cast<void **>(&d->qkv));
    A(B * QD * 4, reinterpret_cast<void **>(&d->attn));
    A(B * H * 4, reinterpret_cast<void **>(&d->o_out));
    A(B * F * 4, reinterpret_cast<void **>(&d->h));
    A(B * H * 4, reinterpret_cast<void **>(&d->f));
    A(B * V * 4, reinterpret_cast<void **>(&d->logits));
    // one workspace for every projection of a step (they run one after the other on one stream)
    // (the tensor-core path's need grows with the token count, the decode path's peaks at 16 tokens)
    size_t need = 0, w = 0;
    for (size_t mm : {B, B > 16 ? (size_t)16 : B}) {
        if (st == BITNET_OK) st = bitnet_bitlinear_fused_workspace_size(mm, H, QD + 2 * KD, BITNET_PATH_AUTO, &w);
        if (w > need) need = w;
        if (st == BITNET_OK) st = bitnet_bitlinear_fused_workspace_size(mm, QD, H, BITNET_PATH_AUTO, &w);
        if (w > need) need = w;
        if (st == BITNET_OK) st = bitnet_bitlinear_fused_workspace_size(mm, H, V, BITNET_PATH_AUTO, &w);
        if (w > need) need = w;
        if (st == BITNET_OK) st = bitnet_ffn_fused_workspace_size(mm, H, F, BITNET_PATH_AUTO, &w);
        if (w > need) need = w;
    }
    d->ws_bytes = align_up(need, 256);
    A(d->ws_bytes, &d->ws);
    d->attn_scratch_bytes = attention_scratch_bytes(B, c.num_heads, c.num_kv_heads, c.head_dim, 32);
    A(d->attn_scratch_bytes, &d->attn_scratch);
    if (st != BITNET_OK) {
        bitnet_decoder_destroy(d);
        return st;
    }
    *out = d;
    return BITNET_OK;
}

static bitnet_status_t upload(bitnet_decoder *d, void *dst, const void *src, size_t bytes)
{
    if (!src) return fail(BITNET_ERR_NULL_POINTER, "decoder: null host buffer");
    return bitnet_backend_copy_to_device(d->backend, dst, src, bytes);
}

extern "C" bitnet_status_t bitnet_decoder_load_embedding(bitnet_decoder *d, const float *table_host)
{
    if (!d) return fail(BITNET_ERR_NULL_POINTER, "bitnet_decoder_load_embedding: null decoder");
    BITNET_CUDA(cudaSetDevice(d->device));
    BITNET_TRY(upload(d, d->embed, table_host, d->cfg.vocab_size * d->cfg.hidden_size * 4));
    d->embed_loaded = true;
    return BITNET_OK;
}

static bitnet_status_t upload_packed(bitnet_decoder *d, uint8_t *dst, const uint8_t *src, size_t n_values)
{
    const size_t bytes = (n_values + 3) / 4;
    BITNET_TRY(upload(d, dst, src, bytes));
    BITNET_TRY(bitnet_sanitize_packed(dst, bytes, nullptr, d->stream));   // code 3 never reaches the kernels
    return BITNET_OK;
}

extern "C" bitnet_status_t bitnet_decoder_load_layer(bitnet_decoder *d, size_t index, const bitnet_decoder_layer *w)
{
    if (!d || !w) return fail(BITNET_ERR_NULL_POINTER, "bitnet_decoder_load_layer: null argument");
    if (index >= d->layers.size()) return fail(BITNET_ERR_INVALID_CONFIG, "layer %zu out of range (have %zu)", index, d->layers.size());
    BITNET_CUDA(cudaSetDevice(d->device));
    const bitnet_decoder_config &c = d->cfg;
    const size_t H = c.hidden_size, QD = q_dim(c), KD = kv_dim(c), F = c.ffn_size;
    DecLayer &L = d->layers[index];
    BITNET_TRY(upload_packed(d, L.qkv, w->q_packed, QD * H));
    BITNET_TRY(upload_packed(d, L.qkv + QD * H / 4, w->k_packed, KD * H));
    BITNET_TRY(upload_packed(d, L.qkv + (QD + KD) * H / 4, w->v_packed, KD * H));
    BITNET_TRY(upload_packed(d, L.o, w->o_packed, H * QD));
    BITNET_TRY(upload_packed(d, L.gate, w->gate_packed, F * H));
    BITNET_TRY(upload_packed(d, L.up, w->up_packed, F * H));
    BITNET_TRY(upload_packed(d, L.down, w->down_packed, H * F));
    BITNET_TRY(upload(d, L.n1w, w->input_norm_weight, H * 4));
    BITNET_TRY(upload(d, L.n1b, w->input_norm_bias, H * 4));
    BITNET_TRY(upload(d, L.n2w, w->post_norm_weight, H * 4));
    BITNET_TRY(upload(d, L.n2b, w->post_norm_bias, H * 4));
    L.s_q = w->q_scale; L.s_k = w->k_scale; L.s_v = w->v_scale; L.s_o = w->o_scale;
    L.s_g = w->gate_scale; L.s_u = w->up_scale; L.s_d = w->down_scale;
    BITNET_CUDA(cudaStreamSynchronize(d->stream));
    L.loaded = true;
    return BITNET_OK;
}

extern "C" bitnet_status_t bitnet_decoder_load_lm_head(bitnet_decoder *d, const uint8_t *packed_host, float scale)
{
    if (!d) return fail(BITNET_ERR_NULL_POINTER, "bitnet_decoder_load_lm_head: null decoder");
    BITNET_CUDA(cudaSetDevice(d->device));
    BITNET_TRY(upload_packed(d, d->lm_head, packed_host, d->cfg.vocab_size * d->cfg.hidden_size));
    BITNET_CUDA(cudaStreamSynchronize(d->stream));
    d->s_lm = scale;
    d->head_loaded = true;
    return BITNET_OK;
}

static bitnet_status_t check_ready(bitnet_decoder *d, size_t B, size_t steps)
{
    if (!d->embed_loaded || !d->head_loaded) return fail(BITNET_ERR_INVALID_CONFIG, "decoder: embedding or language-model head not loaded");
    for (size_t l = 0; l < d->layers.size(); ++l)
        if (!d->layers[l].loaded) return fail(BITNET_ERR_INVALID_CONFIG, "decoder: layer %zu not loaded", l);
    if (B == 0 || B > d->cfg.max_batch) return fail(BITNET_ERR_INCOMPATIBLE_SHAPES, "decoder: batch %zu outside 1..%zu", B, d->cfg.max_batch);
    if (d->batch_in_use && d->batch_in_use != B && d->host_positions)
        return fail(BITNET_ERR_INCOMPATIBLE_SHAPES, "decoder: the cache holds %zu sequences; reset before changing the batch to %zu",
                    d->batch_in_use, B);
    if (d->host_positions + steps > d->cfg.max_seq_len)
        return fail(BITNET_ERR_INCOMPATIBLE_SHAPES, "Sequence length exceeds cache capacity");   // kv_cache.rs:140-142
    return BITNET_OK;
}

extern "C" bitnet_status_t bitnet_decoder_reset(bitnet_decoder *d)
{
    if (!d) return fail(BITNET_ERR_NULL_POINTER, "bitnet_decoder_reset: null decoder");
    std::lock_guard<std::mutex> lock(d->mu);
    BITNET_CUDA(cudaSetDevice(d->device));
    const size_t B = d->cfg.max_batch;
    BITNET_CUDA(cudaMemsetAsync(d->pos, 0, B * 4, d->stream));
    BITNET_CUDA(cudaMemsetAsync(d->finished, 0, B * 4, d->stream));
    BITNET_CUDA(cudaMemsetAsync(d->step_counter, 0, 4, d->stream));
    BITNET_CUDA(cudaStreamSynchronize(d->stream));
    d->host_positions = 0;
    d->batch_in_use = 0;
    d->rng_seeded = false;
    return BITNET_OK;
}

extern "C" bitnet_status_t bitnet_decoder_set_graphs(bitnet_decoder *d, int32_t enabled)
{
    if (!d) return fail(BITNET_ERR_NULL_POINTER, "bitnet_decoder_set_graphs: null decoder");
    d->use_graphs = enabled != 0;
    return BITNET_OK;
}

extern "C" bitnet_status_t bitnet_decoder_feed(bitnet_decoder *d, const int32_t *ids_host, size_t B, size_t T)
{
    if (!d) return fail(BITNET_ERR_NULL_POINTER, "bitnet_decoder_feed: null decoder");
    if (T == 0) return BITNET_OK;
    if (!ids_host) return fail(BITNET_ERR_NULL_POINTER, "bitnet_decoder_feed: null ids");
    std::lock_guard<std::mutex> lock(d->mu);
    BITNET_CUDA(cudaSetDevice(d->device));
    BITNET_TRY(check_ready(d, B, T));
    // [B, T] row-major on the host -> [T][B] on the device, one row per step
    std::vector<int32_t> tb(T * B);
    for (size_t b = 0; b < B; ++b)
        for (size_t t = 0; t < T; ++t) tb[t * B + b] = ids_host[b * T + t];
    BITNET_CUDA(cudaMemcpyAsync(d->feed, tb.data(), T * B * 4, cudaMemcpyHostToDevice, d->stream));
    bitnet_sampling_config sc;
    bitnet_sampling_config_default(&sc);
    for (size_t t = 0; t < T; ++t) {
        BITNET_CUDA(cudaMemcpyAsync(d->ids, d->feed + t * B, B * 4, cudaMemcpyDeviceToDevice, d->stream));
        BITNET_TRY(run_step(d, B, 0, sc, -1));
    }
    BITNET_CUDA(cudaStreamSynchronize(d->stream));
    d->host_positions += T;
    d->batch_in_use = B;
    return BITNET_OK;
}

extern "C" bitnet_status_t bitnet_decoder_decode(bitnet_decoder *d, const int32_t *ids_host, size_t B, size_t n_new,
                                                 const bitnet_sampling_config *sampling, int32_t eos_id,
                                                 int32_t *out_host, size_t *steps_run)
{
    if (!d) return fail(BITNET_ERR_NULL_POINTER, "bitnet_decoder_decode: null decoder");
    if (steps_run) *steps_run = 0;
    if (n_new == 0) return BITNET_OK;
    if (!ids_host || !out_host) return fail(BITNET_ERR_NULL_POINTER, "bitnet_decoder_decode: null buffer");
    std::lock_guard<std::mutex> lock(d->mu);
    BITNET_CUDA(cudaSetDevice(d->device));
    BITNET_TRY(check_ready(d, B, n_new));
    if (n_new > d->history_rows) return fail(BITNET_ERR_INCOMPATIBLE_SHAPES, "decoder: at most %zu new tokens per call", d->history_rows);
    bitnet_sampling_config sc;
    if (sampling) sc = *sampling; else bitnet_sampling_config_default(&sc);
    if (!sc.deterministic && !(sc.temperature > 0.0f)) return fail(BITNET_ERR_INVALID_CONFIG, "Temperature must be positive");
    BITNET_CUDA(cudaMemcpyAsync(d->ids, ids_host, B * 4, cudaMemcpyHostToDevice, d->stream));
    BITNET_CUDA(cudaMemsetAsync(d->step_counter, 0, 4, d->stream));
    if (!d->rng_seeded || d->rng_seed != sc.seed) {   // a new generation, or another seed: sequence i starts from seed + i
        BITNET_TRY(launch_seed_rng(d->rng, B, sc.seed, d->stream));
        d->rng_seeded = true;
        d->rng_seed = sc.seed;
    }
    size_t done = 0;
    std::vector<int32_t> fin(B);
    while (done < n_new) {
        // GenerationState::should_stop (forward_pass_pipeline.rs:322-345) is looked at every 16 steps: the device keeps
        // going in between, a finished sequence repeats its end token
        const size_t burst = eos_id >= 0 ? (n_new - done < 16 ? n_new - done : 16) : n_new - done;
        for (size_t t = 0; t < burst; ++t) BITNET_TRY(run_step(d, B, 1, sc, eos_id));
        done += burst;
        if (eos_id >= 0 && done < n_new) {
            BITNET_CUDA(cudaMemcpyAsync(fin.data(), d->finished, B * 4, cudaMemcpyDeviceToHost, d->stream));
            BITNET_CUDA(cudaStreamSynchronize(d->stream));
            bool all = true;
            for (size_t b = 0; b < B; ++b) all = all && fin[b] != 0;
            if (all) break;
        }
    }
    std::vector<int32_t> hist(done * B);
    BITNET_CUDA(cudaMemcpyAsync(hist.data(), d->history, done * B * 4, cudaMemcpyDeviceToHost, d->stream));
    const cudaError_t err = cudaStreamSynchronize(d->stream);
    if (err != cudaSuccess) return fail(BITNET_ERR_STREAM_SYNC, "stream synchronize: %s", cudaGetErrorString(err));
    for (size_t b = 0; b < B; ++b) {
        for (size_t t = 0; t < done; ++t) out_host[b * n_new + t] = hist[t * B + b];
        for (size_t t = done; t < n_new; ++t) out_host[b * n_new + t] = eos_id;
    }
    d->host_positions += done;
    d->batch_in_use = B;
    if (steps_run) *steps_run = done;
    return BITNET_OK;
}

extern "C" bitnet_status_t bitnet_decoder_generate(bitnet_decoder *d, const int32_t *prompt_host, size_t B, size_t prompt_len,
                                                   size_t max_new_tokens, const bitnet_sampling_config *sampling,
                                                   int32_t eos_id, int32_t *out_host, size_t *steps_run)
{
    if (!d) return fail(BITNET_ERR_NULL_POINTER, "bitnet_decoder_generate: null decoder");
    if (prompt_len == 0) return fail(BITNET_ERR_INCOMPATIBLE_SHAPES, "bitnet_decoder_generate: empty prompt");
    if (!prompt_host) return fail(BITNET_ERR_NULL_POINTER, "bitnet_decoder_generate: null prompt");
    BITNET_TRY(bitnet_decoder_reset(d));
    std::vector<int32_t> ctx(B * (prompt_len - 1)), last(B);
    for (size_t b = 0; b < B; ++b) {
        for (size_t t = 0; t + 1 < prompt_len; ++t) ctx[b * (prompt_len - 1) + t] = prompt_host[b * prompt_len + t];
        last[b] = prompt_host[b * prompt_len + prompt_len - 1];
    }
    BITNET_TRY(bitnet_decoder_feed(d, ctx.data(), B, prompt_len - 1));
    return bitnet_decoder_decode(d, last.data(), B, max_new_tokens, sampling, eos_id, out_host, steps_run);
}

extern "C" bitnet_status_t bitnet_decoder_read(bitnet_decoder *d, int32_t what, void *host, size_t bytes)
{
    if (!d || !host) return fail(BITNET_ERR_NULL_POINTER, "bitnet_decoder_read: null argument");
    BITNET_CUDA(cudaSetDevice(d->device));
    const bitnet_decoder_config &c = d->cfg;
    const void *src = nullptr;
    size_t have = 0;
    switch (what) {
        case BITNET_DECODER_LOGITS: src = d->logits; have = c.max_batch * c.vocab_size * 4; break;
        case BITNET_DECODER_HIDDEN: src = d->x; have = c.max_batch * c.hidden_size * 4; break;
        case BITNET_DECODER_POSITIONS: src = d->pos; have = c.max_batch * 4; break;
        case BITNET_DECODER_KEY_CACHE: src = d->kcache; have = c.num_layers * cache_layer_elems(c) * 2; break;
        case BITNET_DECODER_VALUE_CACHE: src = d->vcache; have = c.num_layers * cache_layer_elems(c) * 2; break;
        default: return fail(BITNET_ERR_INVALID_CONFIG, "bitnet_decoder_read: unknown item %d", what);
    }
    if (bytes > have) return fail(BITNET_ERR_INCOMPATIBLE_SHAPES, "bitnet_decoder_read: %zu bytes asked, %zu held", bytes, have);
    BITNET_CUDA(cudaStreamSynchronize(d->stream));
    BITNET_CUDA(cudaMemcpy(host, src, bytes, cudaMemcpyDeviceToHost));
    return BITNET_OK;
}

// ---- kernel-level entry points of the decode-step pieces ---------------------------------------------------

extern "C" bitnet_status_t bitnet_row_glue_forward(const float *x_dev, size_t M, size_t K, const bitnet_row_glue *glue,
                                                   bitnet_stream_t stream)
{
    if (M == 0) return BITNET_OK;
    if (!x_dev || !glue) return fail(BITNET_ERR_NULL_POINTER, "bitnet_row_glue_forward: null argument");
    RowPre r = {};
    r.residual = glue->residual_dev; r.sum_out = glue->sum_out_dev; r.norm_w = glue->norm_weight_dev; r.norm_b = glue->norm_bias_dev;
    r.eps = glue->norm_eps; r.normed_out = glue->normed_out_dev;
    return launch_row_pre(x_dev, M, K, r, 0, as_stream(stream));
}

extern "C" int32_t bitnet_attention_splits(size_t B, size_t n_kv_heads, size_t max_context)
{
    if (B == 0 || n_kv_heads == 0) return 1;
    return attention_splits(B, n_kv_heads, max_context);
}

extern "C" bitnet_status_t bitnet_attention_scratch_size(size_t B, size_t n_heads, size_t n_kv_heads, size_t head_dim,
                                                         int32_t n_splits, size_t *bytes)
{
    if (!bytes) return fail(BITNET_ERR_NULL_POINTER, "bitnet_attention_scratch_size: null output");
    *bytes = attention_scratch_bytes(B, n_heads, n_kv_heads, head_dim, n_splits < 1 ? 1 : (size_t)n_splits);
    return BITNET_OK;
}

extern "C" bitnet_status_t bitnet_attention_decode(const float *qkv_dev, size_t ldq, size_t k_off, size_t v_off,
                                                   void *k_cache_dev, void *v_cache_dev, const int32_t *pos_dev,
                                                   float *out_dev, size_t B, size_t n_heads, size_t n_kv_heads,
                                                   size_t head_dim, size_t max_seq, int32_t n_splits, void *scratch_dev,
                                                   size_t scratch_bytes, bitnet_stream_t stream)
{
    return launch_attention_decode(qkv_dev, ldq, k_off, v_off, k_cache_dev, v_cache_dev, pos_dev, out_dev, B, n_heads,
                                   n_kv_heads, head_dim, max_seq, n_splits, scratch_dev, scratch_bytes, 0, as_stream(stream));
}

extern "C" bitnet_status_t bitnet_sample_tokens(const float *logits_dev, size_t B, size_t vocab,
                                                const bitnet_sampling_config *cfg, uint64_t *rng_state_dev,
                                                int32_t *next_ids_dev, bitnet_stream_t stream)
{
    bitnet_sampling_config sc;
    if (cfg) sc = *cfg; else bitnet_sampling_config_default(&sc);
    return launch_sample(logits_dev, B, vocab, sc, reinterpret_cast<unsigned long long *>(rng_state_dev), next_ids_dev, nullptr,
                         nullptr, nullptr, nullptr, -1, nullptr, 0, as_stream(stream));
}

extern "C" bitnet_status_t bitnet_seed_sampler(uint64_t *rng_state_dev, size_t B, uint64_t seed, bitnet_stream_t stream)
{
    if (B && !rng_state_dev) return fail(BITNET_ERR_NULL_POINTER, "bitnet_seed_sampler: null states");
    return launch_seed_rng(reinterpret_cast<unsigned long long *>(rng_state_dev), B, seed, as_stream(stream));
}
