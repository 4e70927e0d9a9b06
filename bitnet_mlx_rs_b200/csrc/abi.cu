// C ABI of the kernel-level entry points: argument checks, dispatch between the kernel
// families, error text.  No kernel lives here.
#include <cstring>
#include <mutex>

#include "common.cuh"

namespace bitnet {

static thread_local char g_last_error[512] = "";

bitnet_status_t fail(bitnet_status_t status, const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
    va_end(ap);
    return status;
}

bitnet_status_t check_cuda(cudaError_t err, const char *what)
{
    if (err == cudaSuccess) return BITNET_OK;
    bitnet_status_t st = BITNET_ERR_CUDA_DRIVER;
    if (err == cudaErrorMemoryAllocation) st = BITNET_ERR_MEMORY_ALLOCATION;
    else if (err == cudaErrorNoDevice || err == cudaErrorInsufficientDriver) st = BITNET_ERR_CUDA_NOT_ENABLED;
    else if (err == cudaErrorInvalidDevice) st = BITNET_ERR_DEVICE;
    return fail(st, "%s: %s (%s)", what, cudaGetErrorString(err), cudaGetErrorName(err));
}

bitnet_status_t check_launch(const char *kernel_name)
{
    const cudaError_t err = cudaGetLastError();
    if (err == cudaSuccess) return BITNET_OK;
    return fail(BITNET_ERR_KERNEL_EXECUTION, "launch of %s failed: %s", kernel_name, cudaGetErrorString(err));
}

int device_sm_count()
{
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

static size_t quant_workspace_bytes(size_t M, size_t K)
{
    // int8 activations [M,K] then fp32 scales [M], each 256-byte aligned
    return align_up(M * K, 256) + align_up(M * sizeof(float), 256);
}

static int resolve_path(int path, size_t M, size_t K, size_t N)
{
    if (path != BITNET_PATH_AUTO) return path;
    if (M <= 16 && decode_supports(M, K, N)) return BITNET_PATH_DECODE;
    // a few dozen tokens: the cluster GEMM, unless the layer is so wide that its one-shot CTAs would run in many waves
    // (the language-model head): the persistent GEMM pipelines those better
    if (M <= 128 && N <= 32768 && midm_can_run(M, K, N, false)) return BITNET_PATH_CLUSTER;
    if (prefill_supports(M, K, N)) return BITNET_PATH_PREFILL;
    return BITNET_PATH_GENERIC;
}

static bitnet_status_t check_workspace(void *ws, size_t have, size_t need)
{
    if (need == 0) return BITNET_OK;
    if (!ws) return fail(BITNET_ERR_WORKSPACE, "workspace of %zu bytes required, none given", need);
    if (reinterpret_cast<uintptr_t>(ws) & 255) return fail(BITNET_ERR_WORKSPACE, "workspace must be 256-byte aligned");
    if (have < need) return fail(BITNET_ERR_WORKSPACE, "workspace too small: %zu < %zu bytes", have, need);
    return BITNET_OK;
}

}  // namespace bitnet

using namespace bitnet;

extern "C" const char *bitnet_last_error_string(void) { return g_last_error; }

extern "C" const char *bitnet_status_string(bitnet_status_t s)
{
    switch (s) {
        case BITNET_OK: return "ok";
        case BITNET_ERR_CUDA_NOT_ENABLED: return "CUDA not available";
        case BITNET_ERR_CUDA_DRIVER: return "CUDA driver error";
        case BITNET_ERR_DEVICE: return "CUDA device error";
        case BITNET_ERR_MEMORY_ALLOCATION: return "CUDA memory allocation failed";
        case BITNET_ERR_KERNEL_EXECUTION: return "CUDA kernel execution failed";
        case BITNET_ERR_INVALID_CONFIG: return "Invalid CUDA configuration";
        case BITNET_ERR_UNSUPPORTED_OPERATION: return "Unsupported CUDA operation";
        case BITNET_ERR_STREAM_SYNC: return "CUDA stream synchronization error";
        case BITNET_ERR_UNSUPPORTED_DTYPE: return "Data type not supported on CUDA device";
        case BITNET_ERR_INCOMPATIBLE_SHAPES: return "Incompatible tensor shapes for CUDA operation";
        case BITNET_ERR_PERFORMANCE: return "CUDA performance below threshold";
        case BITNET_ERR_NULL_POINTER: return "null pointer";
        case BITNET_ERR_WORKSPACE: return "workspace missing, misaligned or too small";
    }
    return "unknown status";
}

// CudaError::is_recoverable, bitnet-cuda/src/error.rs:88-103.
extern "C" int32_t bitnet_is_recoverable(bitnet_status_t s)
{
    switch (s) {
        case BITNET_ERR_MEMORY_ALLOCATION:
        case BITNET_ERR_KERNEL_EXECUTION:
        case BITNET_ERR_STREAM_SYNC:
        case BITNET_ERR_PERFORMANCE:
        case BITNET_ERR_CUDA_DRIVER:
        case BITNET_ERR_WORKSPACE:
            return 1;
        default:
            return 0;
    }
}

extern "C" bitnet_status_t bitnet_device_count(int32_t *count)
{
    if (!count) return fail(BITNET_ERR_NULL_POINTER, "bitnet_device_count: null output");
    int n = 0;
    const cudaError_t err = cudaGetDeviceCount(&n);
    if (err != cudaSuccess) {
        *count = 0;
        cudaGetLastError();
        return fail(BITNET_ERR_CUDA_NOT_ENABLED, "no CUDA device: %s", cudaGetErrorString(err));
    }
    *count = n;
    return BITNET_OK;
}

extern "C" bitnet_status_t bitnet_query_device(int32_t device_id, bitnet_device_info *out)
{
    if (!out) return fail(BITNET_ERR_NULL_POINTER, "bitnet_query_device: null output");
    int32_t n = 0;
    BITNET_TRY(bitnet_device_count(&n));
    if (device_id < 0 || device_id >= n) return fail(BITNET_ERR_DEVICE, "device %d out of range (have %d)", device_id, n);
    cudaDeviceProp prop;
    BITNET_CUDA(cudaGetDeviceProperties(&prop, device_id));
    memset(out, 0, sizeof(*out));
    out->device_id = device_id;
    out->cc_major = prop.major;
    out->cc_minor = prop.minor;
    out->sm_count = prop.multiProcessorCount;
    out->l2_bytes = prop.l2CacheSize;
    out->max_smem_per_block = (int32_t)prop.sharedMemPerBlockOptin;
    strncpy(out->name, prop.name, sizeof(out->name) - 1);
    int prev = 0;
    BITNET_CUDA(cudaGetDevice(&prev));
    BITNET_CUDA(cudaSetDevice(device_id));
    const cudaError_t err = cudaMemGetInfo(&out->free_bytes, &out->total_bytes);
    cudaSetDevice(prev);
    return check_cuda(err, "cudaMemGetInfo");
}

extern "C" bitnet_status_t bitnet_w2a8_gemv(const uint8_t *weights_dev, const int8_t *activations_dev,
                                            int32_t *output_dev, size_t n_out, size_t k_in, bitnet_stream_t stream)
{
    if (n_out == 0) return BITNET_OK;
    if (k_in == 0) return fail(BITNET_ERR_INCOMPATIBLE_SHAPES, "bitnet_w2a8_gemv: k == 0");
    if (!weights_dev || !activations_dev || !output_dev)
        return fail(BITNET_ERR_NULL_POINTER, "bitnet_w2a8_gemv: null buffer");
    if (decode_supports(1, k_in, n_out) && ((reinterpret_cast<uintptr_t>(weights_dev) | reinterpret_cast<uintptr_t>(activations_dev)) & 15) == 0) {
        ForwardArgs a = {};
        a.wp = weights_dev; a.x_i8 = activations_dev; a.acc_out = output_dev;
        a.M = 1; a.K = k_in; a.N = n_out; a.ldy = n_out; a.w_scale = 1.0f;
        return launch_decode(a, as_stream(stream));
    }
    return launch_generic(weights_dev, 1.0f, activations_dev, nullptr, nullptr, output_dev, 1, k_in, n_out, n_out,
                          as_stream(stream));
}

extern "C" void launch_w2a8_gemv_optimized(const uint8_t *weights, const int8_t *activations, int32_t *output,
                                           size_t m, size_t k, bitnet_stream_t stream)
{
    (void)bitnet_w2a8_gemv(weights, activations, output, m, k, stream);
}

// Bytes the stand-alone row glue needs in front of a path that does not fuse it: the fp32 row after
// residual add and normalisation.
static size_t glue_bytes(size_t M, size_t K) { return align_up(M * K * sizeof(float), 256); }

static size_t forward_workspace(size_t M, size_t K, size_t N, int path, bool glue)
{
    switch (resolve_path(path, M, K, N)) {
        case BITNET_PATH_DECODE: return glue ? decode_image_bytes_always(M, K, N, false) : decode_image_bytes(M, K, N, false);
        case BITNET_PATH_PREFILL: return prefill_workspace_bytes(M, K, N) + (glue ? glue_bytes(M, K) : 0);
        case BITNET_PATH_GENERIC: return quant_workspace_bytes(M, K) + (glue ? glue_bytes(M, K) : 0);
        case BITNET_PATH_CLUSTER: return midm_workspace_bytes(M, K);
    }
    return 0;
}

extern "C" bitnet_status_t bitnet_bitlinear_workspace_size(size_t M, size_t K, size_t N, int32_t path, size_t *bytes)
{
    if (!bytes) return fail(BITNET_ERR_NULL_POINTER, "bitnet_bitlinear_workspace_size: null output");
    *bytes = 0;
    if (M == 0 || N == 0) return BITNET_OK;
    if (path < BITNET_PATH_AUTO || path > BITNET_PATH_CLUSTER) return fail(BITNET_ERR_INVALID_CONFIG, "unknown path %d", path);
    *bytes = forward_workspace(M, K, N, path, false);
    return BITNET_OK;
}

extern "C" bitnet_status_t bitnet_bitlinear_fused_workspace_size(size_t M, size_t K, size_t N_total, int32_t path, size_t *bytes)
{
    if (!bytes) return fail(BITNET_ERR_NULL_POINTER, "bitnet_bitlinear_fused_workspace_size: null output");
    *bytes = 0;
    if (M == 0 || N_total == 0) return BITNET_OK;
    if (path < BITNET_PATH_AUTO || path > BITNET_PATH_CLUSTER) return fail(BITNET_ERR_INVALID_CONFIG, "unknown path %d", path);
    *bytes = forward_workspace(M, K, N_total, path, true);
    return BITNET_OK;
}

static RowPre to_row_pre(const bitnet_row_glue *g)
{
    RowPre r = {};
    if (g) {
        r.residual = g->residual_dev; r.sum_out = g->sum_out_dev; r.norm_w = g->norm_weight_dev; r.norm_b = g->norm_bias_dev;
        r.eps = g->norm_eps; r.normed_out = g->normed_out_dev;
    }
    return r;
}
static bool has_glue(const RowPre &r) { return r.residual || r.norm_w; }

// One forward over `n_members` weight matrices stacked along N that share x (n_members = 1: a plain
// BitLinear), with optional row glue in front.  The decode path does all of it in two launches; the other
// paths run the glue as its own launch and the members one after the other on the same quantised input
// semantics (each member quantises the same row again, which gives the same int8 values).
static bitnet_status_t forward_impl(const uint8_t *weights_dev, const size_t *rows, const float *scales, int n_members,
                                    const float *x_dev, const RowPre &pre, float *y_dev, size_t M, size_t K, size_t N,
                                    const bitnet_forward_opts &o, void *workspace_dev, size_t workspace_bytes, cudaStream_t s)
{
    const size_t ldy = o.ldy ? o.ldy : N;
    if (ldy < N) return fail(BITNET_ERR_INCOMPATIBLE_SHAPES, "ldy %zu < N %zu", ldy, N);
    const int path = resolve_path(o.path, M, K, N);
    const bool glue = has_glue(pre);
    if (o.n_peers < 0 || o.n_peers > BITNET_MAX_PEERS)
        return fail(BITNET_ERR_INVALID_CONFIG, "n_peers must be in 0..%d (got %d)", BITNET_MAX_PEERS, o.n_peers);
    if (o.n_peers > 0 && path != BITNET_PATH_DECODE && !(path == BITNET_PATH_PREFILL && n_members == 1 && !o.acc_out_dev))
        return fail(BITNET_ERR_UNSUPPORTED_OPERATION, "peer outputs are written by the decode kernel (M <= 16) and by the persistent GEMM (path prefill)");

    if (path == BITNET_PATH_DECODE) {
        ForwardArgs a = {};
        a.wp = weights_dev; a.w_scale = scales[0]; a.x = x_dev; a.y = y_dev;
        a.acc_out = o.acc_out_dev; a.q_out = o.q_out_dev; a.a_scale_out = o.a_scale_out_dev;
        a.M = M; a.K = K; a.N = N; a.ldy = ldy; a.flags = o.flags; a.stages = o.stages;
        for (int r = 0; r < o.n_peers; ++r) {
            if (!o.y_peers_dev[r]) return fail(BITNET_ERR_NULL_POINTER, "y_peers_dev[%d] is null", r);
            a.y_peers[r] = o.y_peers_dev[r];
        }
        a.n_peers = o.n_peers;
        if (n_members > 1) {
            a.n_seg = n_members - 1;
            a.seg_end[0] = rows[0]; a.seg_scale[0] = scales[1];
            if (n_members > 2) { a.seg_end[1] = rows[0] + rows[1]; a.seg_scale[1] = scales[2]; }
        }
        const size_t need = glue ? decode_image_bytes_always(M, K, N, false) : decode_image_bytes(M, K, N, false);
        if (glue) BITNET_TRY(check_workspace(workspace_dev, workspace_bytes, need));
        if (need && workspace_dev && workspace_bytes >= need && (reinterpret_cast<uintptr_t>(workspace_dev) & 255) == 0) {
            a.image_ws = workspace_dev;     // without workspace the kernel quantises by itself
            a.image_ws_bytes = workspace_bytes;
        }
        if (glue) a.pre = &pre;
        return launch_decode(a, s);
    }

    if (path == BITNET_PATH_CLUSTER) {
        // quantiser launch (with the glue) + one cluster launch over all stacked members
        ForwardArgs a = {};
        a.wp = weights_dev; a.w_scale = scales[0]; a.x = x_dev; a.y = y_dev;
        a.acc_out = o.acc_out_dev; a.q_out = o.q_out_dev; a.a_scale_out = o.a_scale_out_dev;
        a.M = M; a.K = K; a.N = N; a.ldy = ldy; a.flags = o.flags;
        if (n_members > 1) {
            a.n_seg = n_members - 1;
            a.seg_end[0] = rows[0]; a.seg_scale[0] = scales[1];
            if (n_members > 2) { a.seg_end[1] = rows[0] + rows[1]; a.seg_scale[1] = scales[2]; }
        }
        if (glue) a.pre = &pre;
        BITNET_TRY(check_workspace(workspace_dev, workspace_bytes, midm_workspace_bytes(M, K)));
        return launch_midm(a, workspace_dev, workspace_bytes, false, s);
    }

    const size_t path_ws = path == BITNET_PATH_PREFILL ? prefill_workspace_bytes(M, K, N) : quant_workspace_bytes(M, K);
    BITNET_TRY(check_workspace(workspace_dev, workspace_bytes, path_ws + (glue ? glue_bytes(M, K) : 0)));
    char *ws = static_cast<char *>(workspace_dev);
    const float *x_eff = x_dev;
    if (glue) {
        RowPre r = pre;
        float *normed = reinterpret_cast<float *>(ws + path_ws);
        if (r.norm_w) {
            if (!r.normed_out) r.normed_out = normed;
            x_eff = r.normed_out;
        } else {   // residual only: the sum is what the projection reads
            if (!r.sum_out) r.sum_out = normed;
            x_eff = r.sum_out;
        }
        BITNET_TRY(launch_row_pre(x_dev, M, K, r, o.flags, s));
    }
    size_t row0 = 0;
    for (int mbr = 0; mbr < n_members; ++mbr) {
        const size_t n_m = n_members == 1 ? N : rows[mbr];
        const uint8_t *w_m = weights_dev + row0 * K / 4;
        float *y_m = y_dev + row0;
        int32_t *acc_m = o.acc_out_dev ? o.acc_out_dev + row0 : nullptr;
        if (path == BITNET_PATH_PREFILL) {
            if (!prefill_supports(M, K, n_m))
                return fail(BITNET_ERR_UNSUPPORTED_OPERATION, "prefill kernel does not cover M=%zu K=%zu N=%zu", M, K, n_m);
            ForwardArgs a = {};
            a.wp = w_m; a.w_scale = scales[mbr]; a.x = x_eff; a.y = y_m; a.acc_out = acc_m;
            a.q_out = mbr == 0 ? o.q_out_dev : nullptr; a.a_scale_out = mbr == 0 ? o.a_scale_out_dev : nullptr;
            a.M = M; a.K = K; a.N = n_m; a.ldy = ldy; a.flags = o.flags;
            for (int r = 0; r < o.n_peers; ++r) {
                if (!o.y_peers_dev[r]) return fail(BITNET_ERR_NULL_POINTER, "y_peers_dev[%d] is null", r);
                a.y_peers[r] = o.y_peers_dev[r];
            }
            a.n_peers = o.n_peers;
            BITNET_TRY(launch_prefill(a, ws, path_ws, s));
        } else {
            int8_t *q = reinterpret_cast<int8_t *>(ws);
            float *as = reinterpret_cast<float *>(ws + align_up(M * K, 256));
            if (mbr == 0) {
                BITNET_TRY(launch_quantize_rows(x_eff, M, K, q, as, s));
                if (o.q_out_dev) BITNET_CUDA(cudaMemcpyAsync(o.q_out_dev, q, M * K, cudaMemcpyDeviceToDevice, s));
                if (o.a_scale_out_dev) BITNET_CUDA(cudaMemcpyAsync(o.a_scale_out_dev, as, M * sizeof(float), cudaMemcpyDeviceToDevice, s));
            }
            BITNET_TRY(launch_generic(w_m, scales[mbr], q, as, y_m, acc_m, M, K, n_m, ldy, s));
        }
        row0 += n_m;
    }
    return BITNET_OK;
}

extern "C" bitnet_status_t bitnet_bitlinear_forward(const uint8_t *weights_dev, float w_scale, const float *x_dev,
                                                    float *y_dev, size_t M, size_t K, size_t N,
                                                    const bitnet_forward_opts *opts, void *workspace_dev,
                                                    size_t workspace_bytes, bitnet_stream_t stream)
{
    bitnet_forward_opts o = {};
    if (opts) o = *opts;
    if (M == 0 || N == 0) return BITNET_OK;   // empty batch: nothing to do
    if (K == 0) return fail(BITNET_ERR_INCOMPATIBLE_SHAPES, "bitnet_bitlinear_forward: K == 0");
    if (!weights_dev || !x_dev || !y_dev) return fail(BITNET_ERR_NULL_POINTER, "bitnet_bitlinear_forward: null buffer");
    if (o.path < BITNET_PATH_AUTO || o.path > BITNET_PATH_CLUSTER) return fail(BITNET_ERR_INVALID_CONFIG, "unknown path %d", o.path);
    const size_t rows[1] = {N};
    const float scales[1] = {w_scale};
    return forward_impl(weights_dev, rows, scales, 1, x_dev, RowPre{}, y_dev, M, K, N, o, workspace_dev, workspace_bytes,
                        as_stream(stream));
}

extern "C" bitnet_status_t bitnet_bitlinear_forward_fused(const uint8_t *weights_dev, const bitnet_stack *stack,
                                                          const float *x_dev, const bitnet_row_glue *glue, float *y_dev,
                                                          size_t M, size_t K, const bitnet_forward_opts *opts,
                                                          void *workspace_dev, size_t workspace_bytes, bitnet_stream_t stream)
{
    bitnet_forward_opts o = {};
    if (opts) o = *opts;
    if (!stack) return fail(BITNET_ERR_NULL_POINTER, "bitnet_bitlinear_forward_fused: null stack");
    if (stack->n_members < 1 || stack->n_members > 3)
        return fail(BITNET_ERR_INVALID_CONFIG, "a stack holds 1 to 3 weight matrices (got %d)", stack->n_members);
    size_t N = 0;
    for (int i = 0; i < stack->n_members; ++i) {
        if (stack->rows[i] == 0) return fail(BITNET_ERR_INCOMPATIBLE_SHAPES, "stack member %d has no rows", i);
        if (i + 1 < stack->n_members && (stack->rows[i] * K) % 64)
            return fail(BITNET_ERR_INCOMPATIBLE_SHAPES, "stack member %d must end on a 16-byte boundary of the packed stream", i);
        N += stack->rows[i];
    }
    if (M == 0) return BITNET_OK;
    if (K == 0) return fail(BITNET_ERR_INCOMPATIBLE_SHAPES, "bitnet_bitlinear_forward_fused: K == 0");
    if (!weights_dev || !x_dev || !y_dev) return fail(BITNET_ERR_NULL_POINTER, "bitnet_bitlinear_forward_fused: null buffer");
    if (o.path < BITNET_PATH_AUTO || o.path > BITNET_PATH_CLUSTER) return fail(BITNET_ERR_INVALID_CONFIG, "unknown path %d", o.path);
    const RowPre pre = to_row_pre(glue);
    if (pre.norm_w && !pre.norm_b) return fail(BITNET_ERR_NULL_POINTER, "normalisation needs weight and bias");
    return forward_impl(weights_dev, stack->rows, stack->scales, stack->n_members, x_dev, pre, y_dev, M, K, N, o, workspace_dev,
                        workspace_bytes, as_stream(stream));
}

// FFN block.  Workspace: [absmax partials of h, 16 KB][gate and up outputs when the pair is
// not fused][whatever the individual projections need].
static size_t ffn_pair_bytes(size_t M, size_t ffn) { return align_up(M * ffn * sizeof(float), 256); }
static const size_t kAmaxBytes = 256 * 16 * sizeof(unsigned);   // up to 256 CTAs x 16 tokens

static size_t ffn_workspace(size_t M, size_t hidden, size_t ffn, int path, bool glue)
{
    const int p1 = resolve_path(path, M, hidden, ffn), p2 = resolve_path(path, M, ffn, hidden);
    const size_t w1 = forward_workspace(M, hidden, ffn, p1, false), w2 = forward_workspace(M, ffn, hidden, p2, false);
    size_t need = kAmaxBytes + (w1 > w2 ? w1 : w2);
    if (p1 == BITNET_PATH_CLUSTER && midm_can_run(M, hidden, ffn, true))
        need += 0;   // the pair launch gates in its epilogue: no gate/up buffers, the glue rides in its quantiser
    else if (p1 != BITNET_PATH_DECODE || !decode_supports_dual(M, hidden, ffn))
        need += 2 * ffn_pair_bytes(M, ffn) + (glue ? glue_bytes(M, hidden) : 0);
    else
        need += (glue ? decode_image_bytes_always(M, hidden, ffn, true) : decode_image_bytes(M, hidden, ffn, true)) +
                decode_image_bytes(M, ffn, hidden, false);
    return need;
}

extern "C" bitnet_status_t bitnet_ffn_workspace_size(size_t M, size_t hidden, size_t ffn, int32_t path, size_t *bytes)
{
    if (!bytes) return fail(BITNET_ERR_NULL_POINTER, "bitnet_ffn_workspace_size: null output");
    *bytes = 0;
    if (M == 0) return BITNET_OK;
    if (path < BITNET_PATH_AUTO || path > BITNET_PATH_CLUSTER) return fail(BITNET_ERR_INVALID_CONFIG, "unknown path %d", path);
    *bytes = ffn_workspace(M, hidden, ffn, path, false);
    return BITNET_OK;
}

extern "C" bitnet_status_t bitnet_ffn_fused_workspace_size(size_t M, size_t hidden, size_t ffn, int32_t path, size_t *bytes)
{
    if (!bytes) return fail(BITNET_ERR_NULL_POINTER, "bitnet_ffn_fused_workspace_size: null output");
    *bytes = 0;
    if (M == 0) return BITNET_OK;
    if (path < BITNET_PATH_AUTO || path > BITNET_PATH_CLUSTER) return fail(BITNET_ERR_INVALID_CONFIG, "unknown path %d", path);
    *bytes = ffn_workspace(M, hidden, ffn, path, true);
    return BITNET_OK;
}

static bitnet_status_t ffn_impl(const uint8_t *w_gate_dev, float s_gate, const uint8_t *w_up_dev, float s_up,
                                const uint8_t *w_down_dev, float s_down, const float *x_dev, const RowPre &pre, float *h_dev,
                                float *y_dev, size_t M, size_t hidden, size_t ffn, const bitnet_forward_opts &o,
                                void *workspace_dev, size_t workspace_bytes, bitnet_stream_t stream, const char *who)
{
    if (M == 0) return BITNET_OK;
    if (hidden == 0 || ffn == 0) return fail(BITNET_ERR_INCOMPATIBLE_SHAPES, "%s: empty feature dimension", who);
    if (!w_gate_dev || !w_up_dev || !w_down_dev || !x_dev || !h_dev || !y_dev)
        return fail(BITNET_ERR_NULL_POINTER, "%s: null buffer", who);
    if (o.q_out_dev || o.a_scale_out_dev || o.acc_out_dev || o.ldy)
        return fail(BITNET_ERR_INVALID_CONFIG, "%s: per-projection debug outputs are not available", who);
    if (o.path < BITNET_PATH_AUTO || o.path > BITNET_PATH_CLUSTER) return fail(BITNET_ERR_INVALID_CONFIG, "unknown path %d", o.path);
    const bool glue = has_glue(pre);
    BITNET_TRY(check_workspace(workspace_dev, workspace_bytes, ffn_workspace(M, hidden, ffn, o.path, glue)));
    cudaStream_t s = as_stream(stream);
    const int p1 = resolve_path(o.path, M, hidden, ffn), p2 = resolve_path(o.path, M, ffn, hidden);
    char *ws = static_cast<char *>(workspace_dev);
    unsigned *amax = reinterpret_cast<unsigned *>(ws);
    size_t off = kAmaxBytes;

    const bool fused_pair = p1 == BITNET_PATH_DECODE && decode_supports_dual(M, hidden, ffn);
    // the gate/up launch leaves per-CTA absmax keys of h; the down launch folds them instead of re-reading h
    const bool chain_amax = fused_pair && p2 == BITNET_PATH_DECODE && decode_grid(ffn) <= 256;
    if (p1 == BITNET_PATH_CLUSTER && midm_can_run(M, hidden, ffn, true)) {
        // gate and up as the two halves of one cluster launch; its epilogue applies up * relu(gate)^2
        ForwardArgs a = {};
        a.wp = w_gate_dev; a.w_scale = s_gate; a.wp2 = w_up_dev; a.w_scale2 = s_up;
        a.x = x_dev; a.y = h_dev; a.M = M; a.K = hidden; a.N = ffn; a.ldy = ffn; a.flags = o.flags;
        if (glue) a.pre = &pre;
        BITNET_TRY(launch_midm(a, ws + off, workspace_bytes - off, false, s));
    } else if (fused_pair) {
        // gate and up stream through one launch; its epilogue applies up * relu(gate)^2
        ForwardArgs a = {};
        a.wp = w_gate_dev; a.w_scale = s_gate; a.wp2 = w_up_dev; a.w_scale2 = s_up;
        a.x = x_dev; a.y = h_dev; a.M = M; a.K = hidden; a.N = ffn; a.ldy = ffn;
        a.flags = o.flags; a.stages = o.stages;
        a.amax_out = chain_amax ? amax : nullptr;
        a.image_ws = ws + off;
        a.image_ws_bytes = glue ? decode_image_bytes_always(M, hidden, ffn, true) : decode_image_bytes(M, hidden, ffn, true);
        if (a.image_ws_bytes == 0) a.image_ws = nullptr;
        off += a.image_ws_bytes;
        if (glue) a.pre = &pre;
        BITNET_TRY(launch_decode(a, s));
    } else {
        float *gate = reinterpret_cast<float *>(ws + off);
        float *up = reinterpret_cast<float *>(ws + off + ffn_pair_bytes(M, ffn));
        off += 2 * ffn_pair_bytes(M, ffn);
        const float *x_eff = x_dev;
        if (glue) {   // the glue runs once, as its own launch, in front of both projections
            RowPre r = pre;
            float *normed = reinterpret_cast<float *>(ws + off);
            off += glue_bytes(M, hidden);
            if (r.norm_w) { if (!r.normed_out) r.normed_out = normed; x_eff = r.normed_out; }
            else { if (!r.sum_out) r.sum_out = normed; x_eff = r.sum_out; }
            BITNET_TRY(launch_row_pre(x_dev, M, hidden, r, o.flags, s));
        }
        bitnet_forward_opts po = {};
        po.path = p1; po.flags = o.flags;
        BITNET_TRY(bitnet_bitlinear_forward(w_up_dev, s_up, x_eff, up, M, hidden, ffn, &po, ws + off, workspace_bytes - off, stream));
        BITNET_TRY(bitnet_bitlinear_forward(w_gate_dev, s_gate, x_eff, gate, M, hidden, ffn, &po, ws + off, workspace_bytes - off, stream));
        BITNET_TRY(launch_gate_relu2(up, gate, h_dev, M * ffn, s));
    }
    if (chain_amax) {
        ForwardArgs a = {};
        a.wp = w_down_dev; a.w_scale = s_down; a.x = h_dev; a.y = y_dev;
        a.M = M; a.K = ffn; a.N = hidden; a.ldy = hidden; a.flags = o.flags; a.stages = o.stages;
        a.amax_in = amax; a.n_amax_in = decode_grid(ffn);
        a.image_ws = ws + off; a.image_ws_bytes = decode_image_bytes(M, ffn, hidden, false);
        if (a.image_ws_bytes == 0) a.image_ws = nullptr;
        off += a.image_ws_bytes;
        return launch_decode(a, s);
    }
    bitnet_forward_opts po = {};
    po.path = p2; po.flags = o.flags; po.stages = o.stages;
    return bitnet_bitlinear_forward(w_down_dev, s_down, h_dev, y_dev, M, ffn, hidden, &po, ws + off, workspace_bytes - off, stream);
}

extern "C" bitnet_status_t bitnet_ffn_forward(const uint8_t *w_gate_dev, float s_gate, const uint8_t *w_up_dev,
                                              float s_up, const uint8_t *w_down_dev, float s_down,
                                              const float *x_dev, float *h_dev, float *y_dev, size_t M,
                                              size_t hidden, size_t ffn, const bitnet_forward_opts *opts,
                                              void *workspace_dev, size_t workspace_bytes, bitnet_stream_t stream)
{
    bitnet_forward_opts o = {};
    if (opts) o = *opts;
    return ffn_impl(w_gate_dev, s_gate, w_up_dev, s_up, w_down_dev, s_down, x_dev, RowPre{}, h_dev, y_dev, M, hidden, ffn, o,
                    workspace_dev, workspace_bytes, stream, "bitnet_ffn_forward");
}

extern "C" bitnet_status_t bitnet_ffn_forward_fused(const uint8_t *w_gate_dev, float s_gate, const uint8_t *w_up_dev,
                                                    float s_up, const uint8_t *w_down_dev, float s_down,
                                                    const float *x_dev, const bitnet_row_glue *glue, float *h_dev,
                                                    float *y_dev, size_t M, size_t hidden, size_t ffn,
                                                    const bitnet_forward_opts *opts, void *workspace_dev,
                                                    size_t workspace_bytes, bitnet_stream_t stream)
{
    bitnet_forward_opts o = {};
    if (opts) o = *opts;
    const RowPre pre = to_row_pre(glue);
    if (pre.norm_w && !pre.norm_b) return fail(BITNET_ERR_NULL_POINTER, "normalisation needs weight and bias");
    return ffn_impl(w_gate_dev, s_gate, w_up_dev, s_up, w_down_dev, s_down, x_dev, pre, h_dev, y_dev, M, hidden, ffn, o,
                    workspace_dev, workspace_bytes, stream, "bitnet_ffn_forward_fused");
}

// The reference's weight-preparation hook (w2a8_gemv.rs:21, :259): nothing to permute here.
extern "C" bitnet_status_t bitnet_prepare_weights(uint8_t *packed_dev, size_t N, size_t K, int32_t layout_id,
                                                  unsigned long long *count_dev, uint32_t *fast_paths,
                                                  bitnet_stream_t stream)
{
    if (fast_paths) *fast_paths = 0;
    if (layout_id != 0) return fail(BITNET_ERR_INVALID_CONFIG, "unknown weight layout %d (0 = canonical packed stream)", layout_id);
    if (N == 0 || K == 0) return BITNET_OK;
    if (!packed_dev) return fail(BITNET_ERR_NULL_POINTER, "bitnet_prepare_weights: null buffer");
    if (fast_paths) *fast_paths = (decode_supports(1, K, N) ? 1u : 0u) | (prefill_supports(17, K, N) ? 2u : 0u);
    return bitnet_sanitize_packed(packed_dev, (N * K + 3) / 4, count_dev, stream);
}
