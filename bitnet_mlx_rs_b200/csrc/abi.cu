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

extern "C" bitnet_status_t bitnet_bitlinear_workspace_size(size_t M, size_t K, size_t N, int32_t path, size_t *bytes)
{
    if (!bytes) return fail(BITNET_ERR_NULL_POINTER, "bitnet_bitlinear_workspace_size: null output");
    *bytes = 0;
    if (M == 0 || N == 0) return BITNET_OK;
    switch (resolve_path(path, M, K, N)) {
        case BITNET_PATH_DECODE: *bytes = decode_image_bytes(M, K, N, false); return BITNET_OK;
        case BITNET_PATH_PREFILL: *bytes = prefill_workspace_bytes(M, K, N); return BITNET_OK;
        case BITNET_PATH_GENERIC: *bytes = quant_workspace_bytes(M, K); return BITNET_OK;
    }
    return fail(BITNET_ERR_INVALID_CONFIG, "unknown path %d", path);
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
    const size_t ldy = o.ldy ? o.ldy : N;
    if (ldy < N) return fail(BITNET_ERR_INCOMPATIBLE_SHAPES, "ldy %zu < N %zu", ldy, N);

    const int path = resolve_path(o.path, M, K, N);
    ForwardArgs a = {};
    a.wp = weights_dev; a.w_scale = w_scale; a.x = x_dev; a.y = y_dev;
    a.acc_out = o.acc_out_dev; a.q_out = o.q_out_dev; a.a_scale_out = o.a_scale_out_dev;
    a.M = M; a.K = K; a.N = N; a.ldy = ldy; a.flags = o.flags; a.stages = o.stages;
    cudaStream_t s = as_stream(stream);
    if (o.n_peers < 0 || o.n_peers > BITNET_MAX_PEERS)
        return fail(BITNET_ERR_INVALID_CONFIG, "n_peers must be in 0..%d (got %d)", BITNET_MAX_PEERS, o.n_peers);
    if (o.n_peers > 0) {
        if (path != BITNET_PATH_DECODE)
            return fail(BITNET_ERR_UNSUPPORTED_OPERATION, "peer outputs are written by the decode kernel only (M <= 16)");
        for (int r = 0; r < o.n_peers; ++r) {
            if (!o.y_peers_dev[r]) return fail(BITNET_ERR_NULL_POINTER, "y_peers_dev[%d] is null", r);
            a.y_peers[r] = o.y_peers_dev[r];
        }
        a.n_peers = o.n_peers;
    }

    switch (path) {
        case BITNET_PATH_DECODE: {
            const size_t need = decode_image_bytes(M, K, N, false);
            if (need && workspace_dev && workspace_bytes >= need && (reinterpret_cast<uintptr_t>(workspace_dev) & 255) == 0) {
                a.image_ws = workspace_dev;     // without workspace the kernel quantises by itself
                a.image_ws_bytes = workspace_bytes;
            }
            return launch_decode(a, s);
        }
        case BITNET_PATH_PREFILL: {
            if (!prefill_supports(M, K, N))
                return fail(BITNET_ERR_UNSUPPORTED_OPERATION, "prefill kernel does not cover M=%zu K=%zu N=%zu", M, K, N);
            BITNET_TRY(check_workspace(workspace_dev, workspace_bytes, prefill_workspace_bytes(M, K, N)));
            return launch_prefill(a, workspace_dev, workspace_bytes, s);
        }
        case BITNET_PATH_GENERIC: {
            BITNET_TRY(check_workspace(workspace_dev, workspace_bytes, quant_workspace_bytes(M, K)));
            int8_t *q = static_cast<int8_t *>(workspace_dev);
            float *as = reinterpret_cast<float *>(static_cast<char *>(workspace_dev) + align_up(M * K, 256));
            BITNET_TRY(launch_quantize_rows(x_dev, M, K, q, as, s));
            if (o.q_out_dev) BITNET_CUDA(cudaMemcpyAsync(o.q_out_dev, q, M * K, cudaMemcpyDeviceToDevice, s));
            if (o.a_scale_out_dev)
                BITNET_CUDA(cudaMemcpyAsync(o.a_scale_out_dev, as, M * sizeof(float), cudaMemcpyDeviceToDevice, s));
            return launch_generic(weights_dev, w_scale, q, as, y_dev, o.acc_out_dev, M, K, N, ldy, s);
        }
    }
    return fail(BITNET_ERR_INVALID_CONFIG, "unknown path %d", o.path);
}

// FFN block.  Workspace: [absmax partials of h, 16 KB][gate and up outputs when the pair is
// not fused][whatever the individual projections need].
static size_t ffn_pair_bytes(size_t M, size_t ffn) { return align_up(M * ffn * sizeof(float), 256); }
static const size_t kAmaxBytes = 256 * 16 * sizeof(unsigned);   // up to 256 CTAs x 16 tokens

extern "C" bitnet_status_t bitnet_ffn_workspace_size(size_t M, size_t hidden, size_t ffn, int32_t path, size_t *bytes)
{
    if (!bytes) return fail(BITNET_ERR_NULL_POINTER, "bitnet_ffn_workspace_size: null output");
    *bytes = 0;
    if (M == 0) return BITNET_OK;
    const int p1 = resolve_path(path, M, hidden, ffn), p2 = resolve_path(path, M, ffn, hidden);
    size_t w1 = 0, w2 = 0;
    BITNET_TRY(bitnet_bitlinear_workspace_size(M, hidden, ffn, p1, &w1));
    BITNET_TRY(bitnet_bitlinear_workspace_size(M, ffn, hidden, p2, &w2));
    size_t need = kAmaxBytes + (w1 > w2 ? w1 : w2);
    if (p1 != BITNET_PATH_DECODE || !decode_supports_dual(M, hidden, ffn)) need += 2 * ffn_pair_bytes(M, ffn);
    else need += decode_image_bytes(M, hidden, ffn, true) + decode_image_bytes(M, ffn, hidden, false);
    *bytes = need;
    return BITNET_OK;
}

extern "C" bitnet_status_t bitnet_ffn_forward(const uint8_t *w_gate_dev, float s_gate, const uint8_t *w_up_dev,
                                              float s_up, const uint8_t *w_down_dev, float s_down,
                                              const float *x_dev, float *h_dev, float *y_dev, size_t M,
                                              size_t hidden, size_t ffn, const bitnet_forward_opts *opts,
                                              void *workspace_dev, size_t workspace_bytes, bitnet_stream_t stream)
{
    bitnet_forward_opts o = {};
    if (opts) o = *opts;
    if (M == 0) return BITNET_OK;
    if (hidden == 0 || ffn == 0) return fail(BITNET_ERR_INCOMPATIBLE_SHAPES, "bitnet_ffn_forward: empty feature dimension");
    if (!w_gate_dev || !w_up_dev || !w_down_dev || !x_dev || !h_dev || !y_dev)
        return fail(BITNET_ERR_NULL_POINTER, "bitnet_ffn_forward: null buffer");
    if (o.q_out_dev || o.a_scale_out_dev || o.acc_out_dev || o.ldy)
        return fail(BITNET_ERR_INVALID_CONFIG, "bitnet_ffn_forward: per-projection debug outputs are not available");
    size_t need = 0;
    BITNET_TRY(bitnet_ffn_workspace_size(M, hidden, ffn, o.path, &need));
    BITNET_TRY(check_workspace(workspace_dev, workspace_bytes, need));
    cudaStream_t s = as_stream(stream);
    const int p1 = resolve_path(o.path, M, hidden, ffn), p2 = resolve_path(o.path, M, ffn, hidden);
    char *ws = static_cast<char *>(workspace_dev);
    unsigned *amax = reinterpret_cast<unsigned *>(ws);
    size_t off = kAmaxBytes;

    const bool fused_pair = p1 == BITNET_PATH_DECODE && decode_supports_dual(M, hidden, ffn);
    // the gate/up launch leaves per-CTA absmax keys of h; the down launch folds them instead of re-reading h
    const bool chain_amax = fused_pair && p2 == BITNET_PATH_DECODE && decode_grid(ffn) <= 256;
    if (fused_pair) {
        // gate and up stream through one launch; its epilogue applies up * relu(gate)^2
        ForwardArgs a = {};
        a.wp = w_gate_dev; a.w_scale = s_gate; a.wp2 = w_up_dev; a.w_scale2 = s_up;
        a.x = x_dev; a.y = h_dev; a.M = M; a.K = hidden; a.N = ffn; a.ldy = ffn;
        a.flags = o.flags; a.stages = o.stages;
        a.amax_out = chain_amax ? amax : nullptr;
        a.image_ws = ws + off; a.image_ws_bytes = decode_image_bytes(M, hidden, ffn, true);
        if (a.image_ws_bytes == 0) a.image_ws = nullptr;
        off += a.image_ws_bytes;
        BITNET_TRY(launch_decode(a, s));
    } else {
        float *gate = reinterpret_cast<float *>(ws + off);
        float *up = reinterpret_cast<float *>(ws + off + ffn_pair_bytes(M, ffn));
        off += 2 * ffn_pair_bytes(M, ffn);
        bitnet_forward_opts po = {};
        po.path = p1; po.flags = o.flags;
        BITNET_TRY(bitnet_bitlinear_forward(w_up_dev, s_up, x_dev, up, M, hidden, ffn, &po, ws + off, workspace_bytes - off, stream));
        BITNET_TRY(bitnet_bitlinear_forward(w_gate_dev, s_gate, x_dev, gate, M, hidden, ffn, &po, ws + off, workspace_bytes - off, stream));
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
