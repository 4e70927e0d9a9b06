// Host side of the library: the state the reference keeps in its bitnet-cuda crate
// (device, stream pool, memory accounting, kernel counters, weight life cycle), in C++
// behind opaque C handles.  Mirrors CudaBackend (bitnet-cuda/src/backend.rs:40-213),
// CudaMemoryManager (memory.rs:47-186), CudaStream/CudaStreamPool (stream.rs:31-207) and
// W2A8GemvKernel's counters (kernels/w2a8_gemv.rs:63-189).
#include <atomic>
#include <chrono>
#include <cstring>
#include <memory>
#include <mutex>
#include <new>
#include <unordered_map>
#include <vector>

#include "common.cuh"

namespace bitnet {
namespace host {

// CudaMemoryManager: a byte budget over cudaMalloc (memory.rs:79-127).  Allocations are
// zero-filled like alloc_zeros; exceeding the budget is MemoryAllocation, not a CUDA call.
class CudaMemoryManager {
public:
    explicit CudaMemoryManager(size_t pool_size) : pool_size_(pool_size) {}
    ~CudaMemoryManager()
    {
        for (auto &kv : live_) cudaFree(kv.first);
    }
    bitnet_status_t allocate(size_t bytes, void **out)
    {
        if (!out) return fail(BITNET_ERR_NULL_POINTER, "allocate: null output");
        *out = nullptr;
        std::lock_guard<std::mutex> lock(mu_);
        if (allocated_ + bytes > pool_size_)
            return fail(BITNET_ERR_MEMORY_ALLOCATION, "Allocation would exceed pool size: %zu + %zu > %zu", allocated_,
                        bytes, pool_size_);
        void *p = nullptr;
        BITNET_CUDA(cudaMalloc(&p, bytes ? bytes : 1));
        // cudaMemset on device memory may return before the fill has run, and the compute
        // streams here are non-blocking (not ordered with the default stream): finish the fill
        // before anyone can touch the buffer
        cudaError_t err = cudaMemset(p, 0, bytes);
        if (err == cudaSuccess) err = cudaStreamSynchronize(cudaStreamLegacy);
        if (err != cudaSuccess) {
            cudaFree(p);
            return check_cuda(err, "cudaMemset");
        }
        live_[p] = bytes;
        allocated_ += bytes;
        if (allocated_ > peak_) peak_ = allocated_;
        ++count_;
        *out = p;
        return BITNET_OK;
    }
    bitnet_status_t release(void *p)
    {
        if (!p) return BITNET_OK;
        std::lock_guard<std::mutex> lock(mu_);
        auto it = live_.find(p);
        if (it == live_.end()) return fail(BITNET_ERR_INVALID_CONFIG, "free: pointer was not allocated by this backend");
        allocated_ -= it->second;
        live_.erase(it);
        return check_cuda(cudaFree(p), "cudaFree");
    }
    float utilization_percent() const
    {
        return pool_size_ ? (float)allocated_ / (float)pool_size_ * 100.0f : 0.0f;
    }
    size_t allocated() const { return allocated_; }
    size_t pool_size() const { return pool_size_; }
    size_t peak() const { return peak_; }
    uint64_t allocation_count() const { return count_; }

private:
    std::mutex mu_;
    size_t pool_size_;
    size_t allocated_ = 0, peak_ = 0;
    uint64_t count_ = 0;
    std::unordered_map<void *, size_t> live_;
};

// One compute stream with the buffers the host-facing calls stage through.
struct CudaStream {
    cudaStream_t stream = nullptr;
    std::atomic<uint64_t> operation_count{0};
    void *pinned = nullptr;   // host staging, grown on demand
    size_t pinned_bytes = 0;
    void *dev = nullptr;      // device staging (x, h, y) + workspace, grown on demand
    size_t dev_bytes = 0;
    std::mutex mu;            // one host-facing call at a time per stream
    // result of an asynchronous host-buffer call that is still in flight on this stream:
    // `pending_bytes` bytes at `pending_src` (pinned staging) go to `pending_dst` once the stream is idle
    void *pending_dst = nullptr;
    const void *pending_src = nullptr;
    size_t pending_bytes = 0;
};

// Waits for the stream and hands a pending asynchronous result to its host buffer (caller holds s.mu).
static bitnet_status_t deliver_pending(CudaStream &s)
{
    if (!s.pending_dst) return BITNET_OK;
    const cudaError_t err = cudaStreamSynchronize(s.stream);
    void *dst = s.pending_dst;
    s.pending_dst = nullptr;
    if (err != cudaSuccess) return fail(BITNET_ERR_STREAM_SYNC, "stream synchronize: %s", cudaGetErrorString(err));
    memcpy(dst, s.pending_src, s.pending_bytes);
    return BITNET_OK;
}

struct Weights {
    uint8_t *packed_dev = nullptr;
    size_t N = 0, K = 0;
    float w_scale = 1.0f;
    unsigned long long invalid_codes = 0;
};

class CudaBackend {
public:
    bitnet_backend_config cfg;
    int device = 0;
    std::unique_ptr<CudaMemoryManager> memory;
    std::vector<std::unique_ptr<CudaStream>> streams;
    // W2A8GemvKernel counters (w2a8_gemv.rs:69-70, :161-189)
    std::atomic<uint64_t> op_count{0};
    std::atomic<uint64_t> total_time_ns{0};
    std::atomic<uint64_t> total_bytes{0};

    ~CudaBackend()
    {
        cudaSetDevice(device);
        for (auto &s : streams) {
            if (s->stream) cudaStreamSynchronize(s->stream);
            if (s->pinned) cudaFreeHost(s->pinned);
            if (s->dev) memory->release(s->dev);
            if (s->stream) cudaStreamDestroy(s->stream);
        }
    }

    bitnet_status_t stream_at(size_t idx, CudaStream **out)
    {
        if (idx >= streams.size())
            return fail(BITNET_ERR_INVALID_CONFIG, "Stream index %zu out of bounds (max: %zu)", idx, streams.size());
        *out = streams[idx].get();
        return BITNET_OK;
    }

    bitnet_status_t ensure_staging(CudaStream &s, size_t host_bytes, size_t dev_bytes)
    {
        if (host_bytes > s.pinned_bytes) {
            if (s.pinned) cudaFreeHost(s.pinned);
            s.pinned = nullptr;
            s.pinned_bytes = 0;
            BITNET_CUDA(cudaMallocHost(&s.pinned, host_bytes));
            s.pinned_bytes = host_bytes;
        }
        if (dev_bytes > s.dev_bytes) {
            if (s.dev) BITNET_TRY(memory->release(s.dev));
            s.dev = nullptr;
            s.dev_bytes = 0;
            BITNET_TRY(memory->allocate(dev_bytes, &s.dev));
            s.dev_bytes = dev_bytes;
        }
        return BITNET_OK;
    }

    void record(uint64_t ns, uint64_t bytes)
    {
        op_count.fetch_add(1, std::memory_order_relaxed);
        total_time_ns.fetch_add(ns, std::memory_order_relaxed);
        total_bytes.fetch_add(bytes, std::memory_order_relaxed);
    }
};

// W2A8GemvConfig validation (w2a8_gemv.rs:15-38: "must be multiple of 32").
static bitnet_status_t validate_config(const bitnet_backend_config &c)
{
    if (c.num_streams == 0 || c.num_streams > 64)
        return fail(BITNET_ERR_INVALID_CONFIG, "num_streams must be in 1..64 (got %zu)", c.num_streams);
    if (c.w2a8_config.block_size == 0 || c.w2a8_config.block_size % 32 != 0 || c.w2a8_config.block_size > 1024)
        return fail(BITNET_ERR_INVALID_CONFIG, "block_size must be a multiple of 32 in 32..1024 (got %u)",
                    c.w2a8_config.block_size);
    if (c.w2a8_config.grid_strategy < BITNET_GRID_FIXED || c.w2a8_config.grid_strategy > BITNET_GRID_OCCUPANCY)
        return fail(BITNET_ERR_INVALID_CONFIG, "unknown grid strategy %d", c.w2a8_config.grid_strategy);
    if (c.w2a8_config.coalescing_level < BITNET_COALESCE_NONE || c.w2a8_config.coalescing_level > BITNET_COALESCE_AGGRESSIVE)
        return fail(BITNET_ERR_INVALID_CONFIG, "unknown coalescing level %d", c.w2a8_config.coalescing_level);
    return BITNET_OK;
}

static uint64_t now_ns()
{
    return (uint64_t)std::chrono::duration_cast<std::chrono::nanoseconds>(
               std::chrono::steady_clock::now().time_since_epoch()).count();
}

}  // namespace host
}  // namespace bitnet

using namespace bitnet;
using namespace bitnet::host;

struct bitnet_backend { CudaBackend impl; };
struct bitnet_weights { Weights impl; };

extern "C" void bitnet_backend_config_default(bitnet_backend_config *cfg)
{
    if (!cfg) return;
    memset(cfg, 0, sizeof(*cfg));
    cfg->device_id = 0;                                  // backend.rs:27-37
    cfg->memory_pool_size = (size_t)1024 * 1024 * 1024;
    cfg->num_streams = 4;
    cfg->enable_profiling = 0;
    cfg->w2a8_config.block_size = 256;                   // w2a8_gemv.rs:28-38
    cfg->w2a8_config.grid_strategy = BITNET_GRID_DYNAMIC;
    cfg->w2a8_config.grid_fixed = 0;
    cfg->w2a8_config.enable_weight_permutation = 1;
    cfg->w2a8_config.enable_dp4a = 1;
    cfg->w2a8_config.coalescing_level = BITNET_COALESCE_AGGRESSIVE;
}

extern "C" bitnet_status_t bitnet_backend_create(const bitnet_backend_config *cfg, bitnet_backend **out)
{
    if (!out) return fail(BITNET_ERR_NULL_POINTER, "bitnet_backend_create: null output");
    *out = nullptr;
    bitnet_backend_config c;
    if (cfg) c = *cfg; else bitnet_backend_config_default(&c);
    BITNET_TRY(validate_config(c));

    bitnet_device_info info;
    BITNET_TRY(bitnet_query_device((int32_t)c.device_id, &info));
    // The kernels are sm_100a binaries: anything else cannot run them
    // (the reference asks for CC >= 7.5, backend.rs:196-201).
    if (info.cc_major != 10)
        return fail(BITNET_ERR_UNSUPPORTED_OPERATION,
                    "Compute capability %d.%d insufficient for BitNet operations (requires 10.x, sm_100a)",
                    info.cc_major, info.cc_minor);
    const size_t min_memory = (size_t)512 * 1024 * 1024;   // backend.rs:204-210
    if (info.free_bytes < min_memory)
        return fail(BITNET_ERR_MEMORY_ALLOCATION, "Insufficient GPU memory: %zu bytes available, %zu bytes required",
                    info.free_bytes, min_memory);

    BITNET_CUDA(cudaSetDevice((int)c.device_id));
    bitnet_backend *b = new (std::nothrow) bitnet_backend();
    if (!b) return fail(BITNET_ERR_MEMORY_ALLOCATION, "out of host memory");
    b->impl.cfg = c;
    b->impl.device = (int)c.device_id;
    b->impl.memory.reset(new CudaMemoryManager(c.memory_pool_size));
    for (size_t i = 0; i < c.num_streams; ++i) {
        std::unique_ptr<CudaStream> s(new CudaStream());
        const cudaError_t err = cudaStreamCreateWithFlags(&s->stream, cudaStreamNonBlocking);
        if (err != cudaSuccess) {
            delete b;
            return check_cuda(err, "cudaStreamCreateWithFlags");
        }
        b->impl.streams.push_back(std::move(s));
    }
    *out = b;
    return BITNET_OK;
}

extern "C" void bitnet_backend_destroy(bitnet_backend *b) { delete b; }

extern "C" bitnet_status_t bitnet_backend_stream(bitnet_backend *b, size_t index, bitnet_stream_t *out)
{
    if (!b || !out) return fail(BITNET_ERR_NULL_POINTER, "bitnet_backend_stream: null argument");
    CudaStream *s = nullptr;
    BITNET_TRY(b->impl.stream_at(index, &s));
    *out = s->stream;
    return BITNET_OK;
}

extern "C" bitnet_status_t bitnet_backend_synchronize(bitnet_backend *b)
{
    if (!b) return fail(BITNET_ERR_NULL_POINTER, "bitnet_backend_synchronize: null backend");
    BITNET_CUDA(cudaSetDevice(b->impl.device));
    for (auto &s : b->impl.streams) {
        std::lock_guard<std::mutex> lock(s->mu);
        BITNET_TRY(deliver_pending(*s));
        const cudaError_t err = cudaStreamSynchronize(s->stream);
        if (err != cudaSuccess) return fail(BITNET_ERR_STREAM_SYNC, "stream synchronize: %s", cudaGetErrorString(err));
    }
    return BITNET_OK;
}

extern "C" bitnet_status_t bitnet_backend_get_performance_stats(bitnet_backend *b, bitnet_performance_stats *out)
{
    if (!b || !out) return fail(BITNET_ERR_NULL_POINTER, "bitnet_backend_get_performance_stats: null argument");
    const uint64_t n = b->impl.op_count.load();
    const uint64_t ns = b->impl.total_time_ns.load();
    const uint64_t bytes = b->impl.total_bytes.load();
    out->total_w2a8_operations = n;
    out->average_execution_time_us = n ? (float)((double)ns / 1e3 / (double)n) : 0.0f;
    out->memory_utilization_percent = b->impl.memory->utilization_percent();
    // bandwidth from the bytes the calls actually moved (the reference divides a
    // hard-coded 1 MB by the mean time, w2a8_gemv.rs:179-189)
    out->peak_bandwidth_gbps = ns ? (float)((double)bytes / (double)ns) : 0.0f;
    return BITNET_OK;
}

extern "C" bitnet_status_t bitnet_backend_allocate(bitnet_backend *b, size_t bytes, void **dev_ptr)
{
    if (!b) return fail(BITNET_ERR_NULL_POINTER, "bitnet_backend_allocate: null backend");
    BITNET_CUDA(cudaSetDevice(b->impl.device));
    return b->impl.memory->allocate(bytes, dev_ptr);
}

extern "C" bitnet_status_t bitnet_backend_free(bitnet_backend *b, void *dev_ptr)
{
    if (!b) return fail(BITNET_ERR_NULL_POINTER, "bitnet_backend_free: null backend");
    return b->impl.memory->release(dev_ptr);
}

extern "C" bitnet_status_t bitnet_backend_copy_to_device(bitnet_backend *b, void *dst_dev, const void *src_host, size_t bytes)
{
    if (!b) return fail(BITNET_ERR_NULL_POINTER, "bitnet_backend_copy_to_device: null backend");
    if (bytes == 0) return BITNET_OK;
    if (!dst_dev || !src_host) return fail(BITNET_ERR_NULL_POINTER, "bitnet_backend_copy_to_device: null buffer");
    BITNET_CUDA(cudaMemcpy(dst_dev, src_host, bytes, cudaMemcpyHostToDevice));
    return BITNET_OK;
}

extern "C" bitnet_status_t bitnet_backend_copy_to_host(bitnet_backend *b, void *dst_host, const void *src_dev, size_t bytes)
{
    if (!b) return fail(BITNET_ERR_NULL_POINTER, "bitnet_backend_copy_to_host: null backend");
    if (bytes == 0) return BITNET_OK;
    if (!dst_host || !src_dev) return fail(BITNET_ERR_NULL_POINTER, "bitnet_backend_copy_to_host: null buffer");
    BITNET_CUDA(cudaMemcpy(dst_host, src_dev, bytes, cudaMemcpyDeviceToHost));
    return BITNET_OK;
}

extern "C" bitnet_status_t bitnet_backend_memory_usage(bitnet_backend *b, size_t *allocated, size_t *pool_size)
{
    if (!b) return fail(BITNET_ERR_NULL_POINTER, "bitnet_backend_memory_usage: null backend");
    if (allocated) *allocated = b->impl.memory->allocated();
    if (pool_size) *pool_size = b->impl.memory->pool_size();
    return BITNET_OK;
}

// CudaBackend::w2a8_gemv with validate_w2a8_dimensions (backend.rs:129-157, :217-257).
extern "C" bitnet_status_t bitnet_backend_w2a8_gemv(bitnet_backend *b, const uint8_t *weights_dev, size_t weights_len,
                                                    const int8_t *activations_dev, size_t activations_len,
                                                    int32_t *output_dev, size_t output_len, size_t m, size_t k,
                                                    size_t stream_idx)
{
    if (!b) return fail(BITNET_ERR_NULL_POINTER, "bitnet_backend_w2a8_gemv: null backend");
    CudaStream *s = nullptr;
    BITNET_TRY(b->impl.stream_at(stream_idx, &s));
    const size_t expected = (m * k + 3) / 4;
    if (weights_len != expected)
        return fail(BITNET_ERR_INCOMPATIBLE_SHAPES, "Weight tensor size mismatch: expected %zu bytes for %zux%zu matrix, got %zu",
                    expected, m, k, weights_len);
    if (activations_len != k)
        return fail(BITNET_ERR_INCOMPATIBLE_SHAPES, "Activation tensor size mismatch: expected %zu elements, got %zu", k,
                    activations_len);
    if (output_len != m)
        return fail(BITNET_ERR_INCOMPATIBLE_SHAPES, "Output tensor size mismatch: expected %zu elements, got %zu", m,
                    output_len);
    const uint64_t t0 = now_ns();
    BITNET_TRY(bitnet_w2a8_gemv(weights_dev, activations_dev, output_dev, m, k, s->stream));
    if (b->impl.cfg.enable_profiling) {
        // profiling mode times the kernel itself, at the price of a synchronisation
        const cudaError_t err = cudaStreamSynchronize(s->stream);
        if (err != cudaSuccess) return fail(BITNET_ERR_STREAM_SYNC, "stream synchronize: %s", cudaGetErrorString(err));
    }
    b->impl.record(now_ns() - t0, expected + k + 4 * m);
    s->operation_count.fetch_add(1, std::memory_order_relaxed);
    return BITNET_OK;
}

enum UploadKind { UPLOAD_PACKED, UPLOAD_TERNARY, UPLOAD_F32 };

static bitnet_status_t upload_common(bitnet_backend *b, const void *host, UploadKind kind, size_t N, size_t K,
                                     float w_scale, bitnet_weights **out)
{
    const bool is_ternary = kind == UPLOAD_TERNARY;
    if (!b || !out) return fail(BITNET_ERR_NULL_POINTER, "upload: null argument");
    *out = nullptr;
    if (!host) return fail(BITNET_ERR_NULL_POINTER, "upload: null host buffer");
    if (N == 0 || K == 0) return fail(BITNET_ERR_INCOMPATIBLE_SHAPES, "upload: empty weight matrix %zux%zu", N, K);
    BITNET_CUDA(cudaSetDevice(b->impl.device));
    const size_t n_values = N * K, n_bytes = (n_values + 3) / 4;
    void *packed = nullptr, *counter = nullptr, *tmp = nullptr;
    cudaStream_t s = b->impl.streams[0]->stream;
    BITNET_TRY(b->impl.memory->allocate(align_up(n_bytes, 256), &packed));
    bitnet_status_t st = b->impl.memory->allocate(256, &counter);
    if (st == BITNET_OK) {
        if (is_ternary) {
            st = b->impl.memory->allocate(n_values, &tmp);
            if (st == BITNET_OK) st = check_cuda(cudaMemcpyAsync(tmp, host, n_values, cudaMemcpyHostToDevice, s), "upload ternary");
            if (st == BITNET_OK) st = bitnet_pack_ternary(static_cast<const int8_t *>(tmp), n_values, static_cast<uint8_t *>(packed), s);
        } else if (kind == UPLOAD_F32) {
            // full-precision weights: absmean quantisation and packing on the device; the scale comes back with the counter
            size_t wsb = 0;
            bitnet_quantize_pack_weights_workspace_size(n_values, &wsb);
            void *qws = nullptr;
            st = b->impl.memory->allocate(n_values * sizeof(float), &tmp);
            if (st == BITNET_OK) st = b->impl.memory->allocate(wsb, &qws);
            if (st == BITNET_OK) st = check_cuda(cudaMemcpyAsync(tmp, host, n_values * sizeof(float), cudaMemcpyHostToDevice, s), "upload fp32 weights");
            float *scale_dev = reinterpret_cast<float *>(static_cast<char *>(counter) + 128);
            if (st == BITNET_OK) st = bitnet_quantize_pack_weights(static_cast<const float *>(tmp), n_values, static_cast<uint8_t *>(packed), scale_dev, qws, wsb, s);
            if (st == BITNET_OK) st = check_cuda(cudaMemcpyAsync(&w_scale, scale_dev, sizeof(float), cudaMemcpyDeviceToHost, s), "read weight scale");
            if (st == BITNET_OK) st = check_cuda(cudaStreamSynchronize(s), "quantise sync");
            if (qws) b->impl.memory->release(qws);
        } else {
            st = check_cuda(cudaMemcpyAsync(packed, host, n_bytes, cudaMemcpyHostToDevice, s), "upload packed");
        }
    }
    unsigned long long found = 0;
    if (st == BITNET_OK) st = bitnet_sanitize_packed(static_cast<uint8_t *>(packed), n_bytes, static_cast<unsigned long long *>(counter), s);
    if (st == BITNET_OK) st = check_cuda(cudaMemcpyAsync(&found, counter, sizeof(found), cudaMemcpyDeviceToHost, s), "read counter");
    if (st == BITNET_OK) st = check_cuda(cudaStreamSynchronize(s), "upload sync");
    if (tmp) b->impl.memory->release(tmp);
    if (counter) b->impl.memory->release(counter);
    if (st != BITNET_OK) {
        b->impl.memory->release(packed);
        return st;
    }
    // the last partial byte of a ternary upload holds padding codes of 0 (= weight -1 on
    // positions past the end); they are never read as weights because every kernel stops
    // at n_values
    bitnet_weights *w = new (std::nothrow) bitnet_weights();
    if (!w) {
        b->impl.memory->release(packed);
        return fail(BITNET_ERR_MEMORY_ALLOCATION, "out of host memory");
    }
    w->impl.packed_dev = static_cast<uint8_t *>(packed);
    w->impl.N = N;
    w->impl.K = K;
    w->impl.w_scale = w_scale;
    w->impl.invalid_codes = found;
    *out = w;
    return BITNET_OK;
}

extern "C" bitnet_status_t bitnet_backend_upload_packed(bitnet_backend *b, const uint8_t *packed_host, size_t N,
                                                        size_t K, float w_scale, bitnet_weights **out)
{
    return upload_common(b, packed_host, UPLOAD_PACKED, N, K, w_scale, out);
}

extern "C" bitnet_status_t bitnet_backend_upload_f32(bitnet_backend *b, const float *weights_host, size_t N, size_t K,
                                                     bitnet_weights **out)
{
    return upload_common(b, weights_host, UPLOAD_F32, N, K, 1.0f, out);
}

// A ternary tensor as GgufLoader::decode_ternary_weights reads it (bitnet-inference/src/gguf.rs:1089-1165): eight bytes of
// metadata (f32 scale, f32 offset, little endian), then the 2-bit codes in the layout the kernels consume; the payload goes
// to the device as it is (code 3 becomes weight 0 there, as in the reference's decoder).
extern "C" bitnet_status_t bitnet_backend_upload_gguf_ternary(bitnet_backend *b, const uint8_t *tensor_host, size_t tensor_bytes,
                                                              size_t N, size_t K, float *offset_out, bitnet_weights **out)
{
    if (!tensor_host) return fail(BITNET_ERR_NULL_POINTER, "upload: null host buffer");
    const size_t payload = (N * K + 3) / 4;
    if (tensor_bytes < payload + 8)
        return fail(BITNET_ERR_INCOMPATIBLE_SHAPES, "Insufficient packed data for tensor: got %zu bytes, expected at least %zu",
                    tensor_bytes, payload + 8);
    float scale = 1.0f, offset = 0.0f;
    unsigned su = (unsigned)tensor_host[0] | ((unsigned)tensor_host[1] << 8) | ((unsigned)tensor_host[2] << 16) | ((unsigned)tensor_host[3] << 24);
    unsigned ou = (unsigned)tensor_host[4] | ((unsigned)tensor_host[5] << 8) | ((unsigned)tensor_host[6] << 16) | ((unsigned)tensor_host[7] << 24);
    memcpy(&scale, &su, 4);
    memcpy(&offset, &ou, 4);
    if (offset_out) *offset_out = offset;
    return upload_common(b, tensor_host + 8, UPLOAD_PACKED, N, K, scale, out);
}

extern "C" bitnet_status_t bitnet_backend_upload_ternary(bitnet_backend *b, const int8_t *ternary_host, size_t N,
                                                         size_t K, float w_scale, bitnet_weights **out)
{
    return upload_common(b, ternary_host, UPLOAD_TERNARY, N, K, w_scale, out);
}

extern "C" bitnet_status_t bitnet_backend_free_weights(bitnet_backend *b, bitnet_weights *w)
{
    if (!w) return BITNET_OK;
    if (!b) return fail(BITNET_ERR_NULL_POINTER, "bitnet_backend_free_weights: null backend");
    const bitnet_status_t st = b->impl.memory->release(w->impl.packed_dev);
    delete w;
    return st;
}

extern "C" bitnet_status_t bitnet_weights_info(const bitnet_weights *w, size_t *N, size_t *K, float *w_scale,
                                               const uint8_t **packed_dev)
{
    if (!w) return fail(BITNET_ERR_NULL_POINTER, "bitnet_weights_info: null weights");
    if (N) *N = w->impl.N;
    if (K) *K = w->impl.K;
    if (w_scale) *w_scale = w->impl.w_scale;
    if (packed_dev) *packed_dev = w->impl.packed_dev;
    return BITNET_OK;
}

extern "C" bitnet_status_t bitnet_backend_bitlinear_forward(bitnet_backend *b, const bitnet_weights *w, const float *x_dev,
                                                            float *y_dev, size_t M, const bitnet_forward_opts *opts,
                                                            size_t stream_idx)
{
    if (!b || !w) return fail(BITNET_ERR_NULL_POINTER, "bitnet_backend_bitlinear_forward: null argument");
    CudaStream *s = nullptr;
    BITNET_TRY(b->impl.stream_at(stream_idx, &s));
    std::lock_guard<std::mutex> lock(s->mu);
    BITNET_CUDA(cudaSetDevice(b->impl.device));
    size_t ws = 0;
    BITNET_TRY(bitnet_bitlinear_workspace_size(M, w->impl.K, w->impl.N, opts ? opts->path : BITNET_PATH_AUTO, &ws));
    BITNET_TRY(b->impl.ensure_staging(*s, 0, ws));
    const uint64_t t0 = now_ns();
    BITNET_TRY(bitnet_bitlinear_forward(w->impl.packed_dev, w->impl.w_scale, x_dev, y_dev, M, w->impl.K, w->impl.N, opts,
                                        ws ? s->dev : nullptr, ws, s->stream));
    b->impl.record(now_ns() - t0, w->impl.N * w->impl.K / 4 + 4 * M * w->impl.K + 4 * M * w->impl.N);
    s->operation_count.fetch_add(1, std::memory_order_relaxed);
    return BITNET_OK;
}

extern "C" bitnet_status_t bitnet_backend_bitlinear_forward_host(bitnet_backend *b, const bitnet_weights *w,
                                                                 const float *x_host, float *y_host, size_t M,
                                                                 const bitnet_forward_opts *opts, size_t stream_idx)
{
    if (!b || !w) return fail(BITNET_ERR_NULL_POINTER, "bitnet_backend_bitlinear_forward_host: null argument");
    if (M == 0) return BITNET_OK;
    if (!x_host || !y_host) return fail(BITNET_ERR_NULL_POINTER, "bitnet_backend_bitlinear_forward_host: null buffer");
    if (opts && (opts->q_out_dev || opts->a_scale_out_dev || opts->acc_out_dev || opts->ldy))
        return fail(BITNET_ERR_INVALID_CONFIG, "host-buffer forward takes no device outputs");
    CudaStream *s = nullptr;
    BITNET_TRY(b->impl.stream_at(stream_idx, &s));
    std::lock_guard<std::mutex> lock(s->mu);
    BITNET_CUDA(cudaSetDevice(b->impl.device));
    BITNET_TRY(deliver_pending(*s));   // an earlier asynchronous call on this stream still owns the staging buffers
    const size_t K = w->impl.K, N = w->impl.N;
    const size_t xb = align_up(M * K * sizeof(float), 256), yb = align_up(M * N * sizeof(float), 256);
    size_t ws = 0;
    BITNET_TRY(bitnet_bitlinear_workspace_size(M, K, N, opts ? opts->path : BITNET_PATH_AUTO, &ws));
    BITNET_TRY(b->impl.ensure_staging(*s, xb + yb, xb + yb + ws));
    char *pin = static_cast<char *>(s->pinned), *dev = static_cast<char *>(s->dev);
    const uint64_t t0 = now_ns();
    memcpy(pin, x_host, M * K * sizeof(float));
    BITNET_CUDA(cudaMemcpyAsync(dev, pin, M * K * sizeof(float), cudaMemcpyHostToDevice, s->stream));
    BITNET_TRY(bitnet_bitlinear_forward(w->impl.packed_dev, w->impl.w_scale, reinterpret_cast<float *>(dev),
                                        reinterpret_cast<float *>(dev + xb), M, K, N, opts, ws ? dev + xb + yb : nullptr, ws,
                                        s->stream));
    BITNET_CUDA(cudaMemcpyAsync(pin + xb, dev + xb, M * N * sizeof(float), cudaMemcpyDeviceToHost, s->stream));
    const cudaError_t err = cudaStreamSynchronize(s->stream);
    if (err != cudaSuccess) return fail(BITNET_ERR_STREAM_SYNC, "stream synchronize: %s", cudaGetErrorString(err));
    memcpy(y_host, pin + xb, M * N * sizeof(float));
    b->impl.record(now_ns() - t0, N * K / 4 + 4 * M * K + 4 * M * N);
    s->operation_count.fetch_add(1, std::memory_order_relaxed);
    return BITNET_OK;
}

// FFN block on host buffers: x is staged through pinned memory, copied in, the block runs, y is
// copied out -- all on the chosen stream.  wait = true: the call returns when y_host is complete;
// false: it returns once everything is queued, and the result reaches y_host when the stream is next
// joined (deliver_pending).
static bitnet_status_t ffn_forward_host_common(bitnet_backend *b, const bitnet_weights *gate, const bitnet_weights *up,
                                               const bitnet_weights *down, const float *x_host, float *y_host, size_t M,
                                               const bitnet_forward_opts *opts, size_t stream_idx, bool wait, const char *who)
{
    if (!b || !gate || !up || !down) return fail(BITNET_ERR_NULL_POINTER, "%s: null argument", who);
    if (M == 0) return BITNET_OK;
    if (!x_host || !y_host) return fail(BITNET_ERR_NULL_POINTER, "%s: null buffer", who);
    const size_t hidden = gate->impl.K, ffn = gate->impl.N;
    if (up->impl.K != hidden || up->impl.N != ffn || down->impl.K != ffn || down->impl.N != hidden)
        return fail(BITNET_ERR_INCOMPATIBLE_SHAPES, "FFN shapes disagree: gate %zux%zu, up %zux%zu, down %zux%zu", ffn, hidden,
                    up->impl.N, up->impl.K, down->impl.N, down->impl.K);
    CudaStream *s = nullptr;
    BITNET_TRY(b->impl.stream_at(stream_idx, &s));
    std::lock_guard<std::mutex> lock(s->mu);
    BITNET_CUDA(cudaSetDevice(b->impl.device));
    BITNET_TRY(deliver_pending(*s));   // an earlier asynchronous call on this stream still owns the staging buffers
    const size_t xb = align_up(M * hidden * sizeof(float), 256), hb = align_up(M * ffn * sizeof(float), 256);
    size_t ws = 0;
    BITNET_TRY(bitnet_ffn_workspace_size(M, hidden, ffn, opts ? opts->path : BITNET_PATH_AUTO, &ws));
    BITNET_TRY(b->impl.ensure_staging(*s, 2 * xb, 2 * xb + hb + ws));
    char *pin = static_cast<char *>(s->pinned), *dev = static_cast<char *>(s->dev);
    float *x_dev = reinterpret_cast<float *>(dev), *y_dev = reinterpret_cast<float *>(dev + xb);
    float *h_dev = reinterpret_cast<float *>(dev + 2 * xb);
    const uint64_t t0 = now_ns();
    memcpy(pin, x_host, M * hidden * sizeof(float));
    BITNET_CUDA(cudaMemcpyAsync(x_dev, pin, M * hidden * sizeof(float), cudaMemcpyHostToDevice, s->stream));
    BITNET_TRY(bitnet_ffn_forward(gate->impl.packed_dev, gate->impl.w_scale, up->impl.packed_dev, up->impl.w_scale,
                                  down->impl.packed_dev, down->impl.w_scale, x_dev, h_dev, y_dev, M, hidden, ffn, opts,
                                  ws ? dev + 2 * xb + hb : nullptr, ws, s->stream));
    BITNET_CUDA(cudaMemcpyAsync(pin + xb, y_dev, M * hidden * sizeof(float), cudaMemcpyDeviceToHost, s->stream));
    if (wait) {
        const cudaError_t err = cudaStreamSynchronize(s->stream);
        if (err != cudaSuccess) return fail(BITNET_ERR_STREAM_SYNC, "stream synchronize: %s", cudaGetErrorString(err));
        memcpy(y_host, pin + xb, M * hidden * sizeof(float));
    } else {
        s->pending_dst = y_host;
        s->pending_src = pin + xb;
        s->pending_bytes = M * hidden * sizeof(float);
    }
    b->impl.record(now_ns() - t0, 3 * (ffn * hidden / 4) + 4 * M * (2 * hidden + 2 * ffn) + 4 * M * (2 * ffn + hidden));
    s->operation_count.fetch_add(1, std::memory_order_relaxed);
    return BITNET_OK;
}

extern "C" bitnet_status_t bitnet_backend_ffn_forward_host(bitnet_backend *b, const bitnet_weights *gate,
                                                           const bitnet_weights *up, const bitnet_weights *down,
                                                           const float *x_host, float *y_host, size_t M,
                                                           const bitnet_forward_opts *opts, size_t stream_idx)
{
    return ffn_forward_host_common(b, gate, up, down, x_host, y_host, M, opts, stream_idx, true, "bitnet_backend_ffn_forward_host");
}

// Asynchronous form, the reference's usage model for its stream pool (launches are asynchronous per
// stream, CudaBackend::synchronize joins them: bitnet-cuda/src/backend.rs:129-178): y_host is complete
// after bitnet_backend_synchronize, or after the next host-buffer call on the same stream.  x_host may be
// reused at once (it is staged before the call returns).
extern "C" bitnet_status_t bitnet_backend_ffn_forward_host_async(bitnet_backend *b, const bitnet_weights *gate,
                                                                 const bitnet_weights *up, const bitnet_weights *down,
                                                                 const float *x_host, float *y_host, size_t M,
                                                                 const bitnet_forward_opts *opts, size_t stream_idx)
{
    return ffn_forward_host_common(b, gate, up, down, x_host, y_host, M, opts, stream_idx, false,
                                   "bitnet_backend_ffn_forward_host_async");
}

// ---- pinned host memory -------------------------------------------------------------------------------

extern "C" bitnet_status_t bitnet_backend_pin_host(bitnet_backend *b, void *host_ptr, size_t bytes)
{
    if (!b) return fail(BITNET_ERR_NULL_POINTER, "bitnet_backend_pin_host: null backend");
    if (bytes == 0) return BITNET_OK;
    if (!host_ptr) return fail(BITNET_ERR_NULL_POINTER, "bitnet_backend_pin_host: null buffer");
    BITNET_CUDA(cudaSetDevice(b->impl.device));
    BITNET_CUDA(cudaHostRegister(host_ptr, bytes, cudaHostRegisterPortable));
    return BITNET_OK;
}

extern "C" bitnet_status_t bitnet_backend_unpin_host(bitnet_backend *b, void *host_ptr)
{
    if (!b) return fail(BITNET_ERR_NULL_POINTER, "bitnet_backend_unpin_host: null backend");
    if (!host_ptr) return BITNET_OK;
    BITNET_CUDA(cudaHostUnregister(host_ptr));
    return BITNET_OK;
}

// ---- a fixed batch of FFN blocks as one replayable unit -------------------------------------------------

namespace {

bool host_ptr_is_pinned(const void *p)
{
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return attr.type == cudaMemoryTypeHost;
}

// One piece (at most 8 KB) of a copy between page-locked host memory, through its device alias, and device memory.
struct CopyChunk {
    const uint4 *src;
    uint4 *dst;
    unsigned units;   // 16-byte units
};

// Many small host<->device copies as one launch: the SMs move the bytes over the host link themselves (every
// 16-byte unit is one request in flight), where a copy-engine transfer per buffer costs microseconds each.
__global__ void __launch_bounds__(256) plan_copy_kernel(const CopyChunk *__restrict__ chunks)
{
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const CopyChunk c = chunks[blockIdx.x];
    for (unsigned u = threadIdx.x; u < c.units; u += 256) c.dst[u] = c.src[u];
}

struct PlanCall {
    const Weights *gate, *up, *down;
    size_t M;
    const float *x_host;
    float *y_host;
    bool x_pinned, y_pinned;
    const float *x_src;   // what the in-graph copy reads: the caller's pinned buffer or this plan's staging
    float *y_dst;
    float *x_dev, *h_dev, *y_dev;
    const float *x_src_alias;   // device-side aliases of x_src / y_dst (null when the host memory is not mapped)
    float *y_dst_alias;
    void *ws;
    size_t ws_bytes;
};

}  // namespace

struct bitnet_ffn_plan {
    bitnet_backend *backend = nullptr;
    std::vector<PlanCall> calls;
    void *dev_slab = nullptr;
    void *pin_slab = nullptr;
    std::vector<cudaStream_t> lanes;   // lanes[0] is the stream the graph is launched on
    std::vector<cudaEvent_t> events;
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    bitnet_forward_opts opts = {};
    std::mutex mu;
    size_t bytes_per_run = 0;
    // Equal shapes and at most 16 tokens per call: the calls run as a few grouped launches (bitnet_ffn_group_*)
    // instead of two to four launches each; groups[g] covers calls [group_first[g], group_first[g + 1]).
    std::vector<bitnet_ffn_group *> groups;
    std::vector<size_t> group_first;
    std::vector<cudaEvent_t> group_events;   // per group: one per lane (its inputs are on the device), then one (its kernels are done)
    // When every bound host buffer is mapped into the device's address space, a group's inputs and outputs move
    // by one copy launch each (plan_copy_kernel) instead of one copy-engine transfer per buffer.
    CopyChunk *chunks_dev = nullptr;
    std::vector<unsigned> in_first, in_count, out_first, out_count;   // per group: its chunks in chunks_dev
};

static void plan_release(bitnet_ffn_plan *p)
{
    if (!p) return;
    if (p->backend) cudaSetDevice(p->backend->impl.device);
    if (!p->lanes.empty()) cudaStreamSynchronize(p->lanes[0]);
    if (p->exec) cudaGraphExecDestroy(p->exec);
    if (p->graph) cudaGraphDestroy(p->graph);
    for (cudaEvent_t e : p->events) cudaEventDestroy(e);
    for (cudaEvent_t e : p->group_events) cudaEventDestroy(e);
    for (bitnet_ffn_group *g : p->groups) bitnet_ffn_group_destroy(g);
    if (p->chunks_dev) cudaFree(p->chunks_dev);
    for (cudaStream_t s : p->lanes) cudaStreamDestroy(s);
    if (p->pin_slab) cudaFreeHost(p->pin_slab);
    if (p->dev_slab && p->backend) p->backend->impl.memory->release(p->dev_slab);
    delete p;
}

// Queues every call of the plan on its lane: copy in, FFN block, copy out.  Used once eagerly (which
// also sets every launch attribute outside the capture) and once under stream capture.
static bitnet_status_t plan_enqueue(bitnet_ffn_plan *p)
{
    const size_t L = p->lanes.size();
    cudaStream_t origin = p->lanes[0];
    BITNET_CUDA(cudaEventRecord(p->events[0], origin));
    for (size_t l = 1; l < L; ++l) BITNET_CUDA(cudaStreamWaitEvent(p->lanes[l], p->events[0], 0));
    if (!p->groups.empty()) {
        // Every input copy is queued first, dealt to the lanes; group g starts on the origin stream when ITS inputs
        // have landed (later groups' copies keep running beside its kernels), and its outputs leave on the lanes
        // while the next group computes.
        const size_t G = p->groups.size();
        auto ev = [&](size_t g, size_t k) { return p->group_events[g * (L + 1) + k]; };
        if (p->chunks_dev) {
            // copy launches: inputs of all groups on one lane, kernels on the origin stream, outputs on another lane
            cudaStream_t in_s = L > 1 ? p->lanes[1] : origin, out_s = L > 2 ? p->lanes[2] : in_s;
            auto copy = [&](unsigned first, unsigned count, cudaStream_t s) -> bitnet_status_t {
                BITNET_CUDA(cudaGetLastError());
                plan_copy_kernel<<<count, 256, 0, s>>>(p->chunks_dev + first);
                BITNET_CUDA(cudaGetLastError());
                return BITNET_OK;
            };
            for (size_t g = 0; g < G; ++g) {
                BITNET_TRY(copy(p->in_first[g], p->in_count[g], in_s));
                if (in_s != origin) BITNET_CUDA(cudaEventRecord(ev(g, 1), in_s));
            }
            for (size_t g = 0; g < G; ++g) {
                if (in_s != origin) BITNET_CUDA(cudaStreamWaitEvent(origin, ev(g, 1), 0));
                BITNET_TRY(bitnet_ffn_group_run(p->groups[g], origin));
                if (out_s != origin) {
                    BITNET_CUDA(cudaEventRecord(ev(g, L), origin));
                    BITNET_CUDA(cudaStreamWaitEvent(out_s, ev(g, L), 0));
                }
                BITNET_TRY(copy(p->out_first[g], p->out_count[g], out_s));
            }
            for (size_t l = 1; l < L; ++l) {
                BITNET_CUDA(cudaEventRecord(p->events[l], p->lanes[l]));
                BITNET_CUDA(cudaStreamWaitEvent(origin, p->events[l], 0));
            }
            return BITNET_OK;
        }
        // the origin stream carries the kernels; copies go to the other lanes when there are any
        auto copy_lane = [&](size_t i) { return L > 1 ? p->lanes[1 + i % (L - 1)] : origin; };
        for (size_t g = 0; g < G; ++g) {
            for (size_t i = p->group_first[g]; i < p->group_first[g + 1]; ++i) {
                const PlanCall &c = p->calls[i];
                BITNET_CUDA(cudaMemcpyAsync(c.x_dev, c.x_src, c.M * c.gate->K * sizeof(float), cudaMemcpyHostToDevice, copy_lane(i)));
            }
            for (size_t l = 1; l < L; ++l) BITNET_CUDA(cudaEventRecord(ev(g, l), p->lanes[l]));
        }
        for (size_t g = 0; g < G; ++g) {
            for (size_t l = 1; l < L; ++l) BITNET_CUDA(cudaStreamWaitEvent(origin, ev(g, l), 0));
            BITNET_TRY(bitnet_ffn_group_run(p->groups[g], origin));
            BITNET_CUDA(cudaEventRecord(ev(g, L), origin));
            for (size_t l = 1; l < L; ++l) BITNET_CUDA(cudaStreamWaitEvent(p->lanes[l], ev(g, L), 0));
            for (size_t i = p->group_first[g]; i < p->group_first[g + 1]; ++i) {
                const PlanCall &c = p->calls[i];
                BITNET_CUDA(cudaMemcpyAsync(c.y_dst, c.y_dev, c.M * c.gate->K * sizeof(float), cudaMemcpyDeviceToHost, copy_lane(i)));
            }
        }
        for (size_t l = 1; l < L; ++l) {
            BITNET_CUDA(cudaEventRecord(p->events[l], p->lanes[l]));
            BITNET_CUDA(cudaStreamWaitEvent(origin, p->events[l], 0));
        }
        return BITNET_OK;
    }
    for (size_t i = 0; i < p->calls.size(); ++i) {
        const PlanCall &c = p->calls[i];
        cudaStream_t s = p->lanes[i % L];
        const size_t hidden = c.gate->K, ffn = c.gate->N;
        BITNET_CUDA(cudaMemcpyAsync(c.x_dev, c.x_src, c.M * hidden * sizeof(float), cudaMemcpyHostToDevice, s));
        BITNET_TRY(bitnet_ffn_forward(c.gate->packed_dev, c.gate->w_scale, c.up->packed_dev, c.up->w_scale, c.down->packed_dev,
                                      c.down->w_scale, c.x_dev, c.h_dev, c.y_dev, c.M, hidden, ffn, &p->opts, c.ws, c.ws_bytes, s));
        BITNET_CUDA(cudaMemcpyAsync(c.y_dst, c.y_dev, c.M * hidden * sizeof(float), cudaMemcpyDeviceToHost, s));
    }
    for (size_t l = 1; l < L; ++l) {
        BITNET_CUDA(cudaEventRecord(p->events[l], p->lanes[l]));
        BITNET_CUDA(cudaStreamWaitEvent(origin, p->events[l], 0));
    }
    return BITNET_OK;
}

// Groups the plan's calls when they qualify (one shape, at most 16 tokens each, automatic path); otherwise the plan
// keeps its per-call launches.  Three groups at most, of a few dozen calls each: a group's four launches cost a
// fixed twenty-odd microseconds, and more groups let copies of one overlap the kernels of another.
static bitnet_status_t plan_build_groups(bitnet_ffn_plan *p)
{
    const size_t n = p->calls.size();
    if (n < 2 || (p->opts.path != BITNET_PATH_AUTO && p->opts.path != BITNET_PATH_DECODE)) return BITNET_OK;
    const size_t hidden = p->calls[0].gate->K, ffn = p->calls[0].gate->N;
    for (const PlanCall &c : p->calls)
        if (c.gate->K != hidden || c.gate->N != ffn || c.M > 16) return BITNET_OK;
    if (hidden % 64 || ffn % 64 || hidden > 8192 || ffn > 16384) return BITNET_OK;
    size_t G = n / 24;
    if (G < 1) G = 1;
    if (G > 3) G = 3;
    const size_t L = p->lanes.size();
    std::vector<bitnet_ffn_group_member> members(n);
    for (size_t i = 0; i < n; ++i) {
        const PlanCall &c = p->calls[i];
        members[i] = bitnet_ffn_group_member{static_cast<const uint8_t *>(c.gate->packed_dev), static_cast<const uint8_t *>(c.up->packed_dev),
                                             static_cast<const uint8_t *>(c.down->packed_dev), c.gate->w_scale, c.up->w_scale, c.down->w_scale,
                                             c.x_dev, c.y_dev, c.M};
    }
    for (size_t g = 0; g <= G; ++g) p->group_first.push_back(g * n / G);
    for (size_t g = 0; g < G; ++g) {
        bitnet_ffn_group *grp = nullptr;
        const bitnet_status_t st = bitnet_ffn_group_create(members.data() + p->group_first[g], p->group_first[g + 1] - p->group_first[g], hidden, ffn, &grp);
        if (st == BITNET_ERR_UNSUPPORTED_OPERATION) {   // this shape has no grouped kernel: per-call launches
            for (bitnet_ffn_group *q : p->groups) bitnet_ffn_group_destroy(q);
            p->groups.clear();
            p->group_first.clear();
            return BITNET_OK;
        }
        if (st != BITNET_OK) return st;
        p->groups.push_back(grp);
    }
    for (size_t k = 0; k < G * (L + 1); ++k) {
        cudaEvent_t e = nullptr;
        BITNET_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        p->group_events.push_back(e);
    }
    // copy launches need every host buffer mapped for the device (page-locked memory normally is)
    bool mapped = true;
    for (PlanCall &c : p->calls) {
        void *dx = nullptr, *dy = nullptr;
        if (cudaHostGetDevicePointer(&dx, const_cast<float *>(c.x_src), 0) != cudaSuccess ||
            cudaHostGetDevicePointer(&dy, c.y_dst, 0) != cudaSuccess || (reinterpret_cast<uintptr_t>(dx) & 15) || (reinterpret_cast<uintptr_t>(dy) & 15)) {
            cudaGetLastError();
            mapped = false;
            break;
        }
        c.x_src_alias = static_cast<const float *>(dx);
        c.y_dst_alias = static_cast<float *>(dy);
    }
    if (!mapped) return BITNET_OK;
    std::vector<CopyChunk> chunks;
    const unsigned per_chunk = 512;   // 8 KB
    auto add = [&](const float *src, float *dst, size_t bytes) {
        const size_t units = bytes / 16;   // hidden % 64 == 0: a row is a whole number of units
        for (size_t u = 0; u < units; u += per_chunk)
            chunks.push_back(CopyChunk{reinterpret_cast<const uint4 *>(src) + u, reinterpret_cast<uint4 *>(dst) + u,
                                       (unsigned)(units - u < per_chunk ? units - u : per_chunk)});
    };
    for (size_t g = 0; g < G; ++g) {
        p->in_first.push_back((unsigned)chunks.size());
        for (size_t i = p->group_first[g]; i < p->group_first[g + 1]; ++i) add(p->calls[i].x_src_alias, p->calls[i].x_dev, p->calls[i].M * hidden * sizeof(float));
        p->in_count.push_back((unsigned)chunks.size() - p->in_first[g]);
        p->out_first.push_back((unsigned)chunks.size());
        for (size_t i = p->group_first[g]; i < p->group_first[g + 1]; ++i) add(p->calls[i].y_dev, p->calls[i].y_dst_alias, p->calls[i].M * hidden * sizeof(float));
        p->out_count.push_back((unsigned)chunks.size() - p->out_first[g]);
    }
    BITNET_CUDA(cudaMalloc(reinterpret_cast<void **>(&p->chunks_dev), chunks.size() * sizeof(CopyChunk)));
    BITNET_CUDA(cudaMemcpy(p->chunks_dev, chunks.data(), chunks.size() * sizeof(CopyChunk), cudaMemcpyHostToDevice));
    return BITNET_OK;
}

extern "C" bitnet_status_t bitnet_backend_ffn_plan_create(bitnet_backend *b, const bitnet_ffn_call *calls, size_t n_calls,
                                                          const bitnet_forward_opts *opts, size_t n_lanes,
                                                          bitnet_ffn_plan **out)
{
    if (!b || !out) return fail(BITNET_ERR_NULL_POINTER, "bitnet_backend_ffn_plan_create: null argument");
    *out = nullptr;
    if (n_calls == 0 || !calls) return fail(BITNET_ERR_INVALID_CONFIG, "bitnet_backend_ffn_plan_create: no calls");
    if (opts && (opts->q_out_dev || opts->a_scale_out_dev || opts->acc_out_dev || opts->ldy || opts->n_peers))
        return fail(BITNET_ERR_INVALID_CONFIG, "an FFN plan takes no device outputs");
    if (n_lanes == 0) n_lanes = 8;
    if (n_lanes > n_calls) n_lanes = n_calls;
    if (n_lanes > 32) n_lanes = 32;
    BITNET_CUDA(cudaSetDevice(b->impl.device));

    bitnet_ffn_plan *p = new (std::nothrow) bitnet_ffn_plan();
    if (!p) return fail(BITNET_ERR_MEMORY_ALLOCATION, "out of host memory");
    p->backend = b;
    if (opts) p->opts = *opts;
    // blocks of different lanes share the SMs: small CTAs, launches chained inside a lane
    if (n_lanes > 1) p->opts.flags |= BITNET_FLAG_THROUGHPUT;
    p->opts.flags |= BITNET_FLAG_PDL;

    size_t dev_bytes = 0, pin_bytes = 0;
    bitnet_status_t st = BITNET_OK;
    p->calls.resize(n_calls);
    for (size_t i = 0; i < n_calls && st == BITNET_OK; ++i) {
        const bitnet_ffn_call &in = calls[i];
        PlanCall &c = p->calls[i];
        if (!in.gate || !in.up || !in.down || !in.x_host || !in.y_host || in.M == 0) {
            st = fail(BITNET_ERR_NULL_POINTER, "FFN plan: call %zu has a null member or no tokens", i);
            break;
        }
        c.gate = &in.gate->impl; c.up = &in.up->impl; c.down = &in.down->impl;
        c.M = in.M; c.x_host = in.x_host; c.y_host = in.y_host;
        const size_t hidden = c.gate->K, ffn = c.gate->N;
        if (c.up->K != hidden || c.up->N != ffn || c.down->K != ffn || c.down->N != hidden) {
            st = fail(BITNET_ERR_INCOMPATIBLE_SHAPES, "FFN plan: shapes of call %zu disagree", i);
            break;
        }
        c.x_pinned = host_ptr_is_pinned(c.x_host);
        c.y_pinned = host_ptr_is_pinned(c.y_host);
        const size_t xb = align_up(c.M * hidden * sizeof(float), 256), hb = align_up(c.M * ffn * sizeof(float), 256);
        st = bitnet_ffn_workspace_size(c.M, hidden, ffn, p->opts.path, &c.ws_bytes);
        dev_bytes += 2 * xb + hb + align_up(c.ws_bytes, 256);
        pin_bytes += (c.x_pinned ? 0 : xb) + (c.y_pinned ? 0 : xb);
        p->bytes_per_run += 3 * (ffn * hidden / 4) + 4 * c.M * (2 * hidden + 2 * ffn) + 4 * c.M * (2 * ffn + hidden);
    }
    if (st == BITNET_OK) st = b->impl.memory->allocate(dev_bytes, &p->dev_slab);
    if (st == BITNET_OK && pin_bytes) st = check_cuda(cudaMallocHost(&p->pin_slab, pin_bytes), "cudaMallocHost");
    if (st == BITNET_OK) {
        char *dev = static_cast<char *>(p->dev_slab), *pin = static_cast<char *>(p->pin_slab);
        for (PlanCall &c : p->calls) {
            const size_t hidden = c.gate->K, ffn = c.gate->N;
            const size_t xb = align_up(c.M * hidden * sizeof(float), 256), hb = align_up(c.M * ffn * sizeof(float), 256);
            c.x_dev = reinterpret_cast<float *>(dev); dev += xb;
            c.y_dev = reinterpret_cast<float *>(dev); dev += xb;
            c.h_dev = reinterpret_cast<float *>(dev); dev += hb;
            c.ws = c.ws_bytes ? dev : nullptr; dev += align_up(c.ws_bytes, 256);
            if (c.x_pinned) c.x_src = c.x_host; else { c.x_src = reinterpret_cast<float *>(pin); pin += xb; }
            if (c.y_pinned) c.y_dst = c.y_host; else { c.y_dst = reinterpret_cast<float *>(pin); pin += xb; }
        }
        for (size_t l = 0; l < n_lanes && st == BITNET_OK; ++l) {
            cudaStream_t s = nullptr;
            cudaEvent_t e = nullptr;
            st = check_cuda(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking), "cudaStreamCreateWithFlags");
            if (st == BITNET_OK) p->lanes.push_back(s);
            if (st == BITNET_OK) st = check_cuda(cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "cudaEventCreateWithFlags");
            if (st == BITNET_OK) p->events.push_back(e);
        }
    }
    if (st == BITNET_OK) st = plan_build_groups(p);
    // once eagerly (sets launch attributes, checks every call), then the same thing as a graph
    if (st == BITNET_OK) st = plan_enqueue(p);
    if (st == BITNET_OK) st = check_cuda(cudaStreamSynchronize(p->lanes[0]), "FFN plan: first run");
    // with programmatic dependent launch inside the lanes first; if this driver cannot capture or
    // instantiate that, with ordinary dependencies
    for (int attempt = 0; st == BITNET_OK && attempt < 2 && !p->exec; ++attempt) {
        if (attempt == 1) p->opts.flags &= ~BITNET_FLAG_PDL;
        bitnet_status_t cs = check_cuda(cudaStreamBeginCapture(p->lanes[0], cudaStreamCaptureModeThreadLocal), "cudaStreamBeginCapture");
        if (cs == BITNET_OK) {
            const bitnet_status_t q = plan_enqueue(p);
            const cudaError_t err = cudaStreamEndCapture(p->lanes[0], &p->graph);   // always end the capture
            cs = q != BITNET_OK ? q : check_cuda(err, "cudaStreamEndCapture");
        }
        if (cs == BITNET_OK) cs = check_cuda(cudaGraphInstantiate(&p->exec, p->graph, 0), "cudaGraphInstantiate");
        if (cs != BITNET_OK) {
            cudaGetLastError();
            if (p->exec) { cudaGraphExecDestroy(p->exec); p->exec = nullptr; }
            if (p->graph) { cudaGraphDestroy(p->graph); p->graph = nullptr; }
            if (attempt == 1) st = cs;
        }
    }
    if (st != BITNET_OK) {
        cudaGetLastError();
        plan_release(p);
        return st;
    }
    *out = p;
    return BITNET_OK;
}

extern "C" bitnet_status_t bitnet_backend_ffn_plan_run(bitnet_ffn_plan *p)
{
    if (!p) return fail(BITNET_ERR_NULL_POINTER, "bitnet_backend_ffn_plan_run: null plan");
    std::lock_guard<std::mutex> lock(p->mu);
    BITNET_CUDA(cudaSetDevice(p->backend->impl.device));
    const uint64_t t0 = now_ns();
    for (const PlanCall &c : p->calls)
        if (!c.x_pinned) memcpy(const_cast<float *>(c.x_src), c.x_host, c.M * c.gate->K * sizeof(float));
    BITNET_CUDA(cudaGraphLaunch(p->exec, p->lanes[0]));
    const cudaError_t err = cudaStreamSynchronize(p->lanes[0]);
    if (err != cudaSuccess) return fail(BITNET_ERR_STREAM_SYNC, "stream synchronize: %s", cudaGetErrorString(err));
    for (const PlanCall &c : p->calls)
        if (!c.y_pinned) memcpy(c.y_host, c.y_dst, c.M * c.gate->K * sizeof(float));
    p->backend->impl.record(now_ns() - t0, p->bytes_per_run);
    return BITNET_OK;
}

extern "C" void bitnet_backend_ffn_plan_destroy(bitnet_ffn_plan *p) { plan_release(p); }
