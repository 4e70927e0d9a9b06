// bitnet_bitlinear_forward_static: the decode-path BitLinear forward for callers that can neither
// allocate device memory nor hand over a workspace.
//
// Who that is: a host loop that runs inside a fixed memory budget decided at start-up (every
// byte of the device already belongs to weights, KV cache and I/O buffers), a plug-in that is
// called while its host application is capturing a stream or otherwise forbids allocation
// calls, or a binding whose ownership rules make "lend me N bytes of scratch" awkward to
// express.  For them the scratch the decode path needs -- the once-quantised activations that
// all CTAs of the kernel fetch -- lives in a fixed array inside the library image.
//
// Cost and limits: every GPU that loads the library keeps BITNET_STATIC_SCRATCH_BYTES
// (136 KiB) resident until the process exits.  The array is shared by all calls on a device:
// two calls that can overlap on the GPU (different streams, no dependency) race on it.  It keeps
// the previous call's bytes, and nothing in it has to start at zero: the quantiser overwrites
// every byte that stands for a real token and a real k, and the stale remainder is of two kinds,
// both harmless.  Rows of tokens that do not exist feed accumulator columns that are never
// written.  Fragment slots of k chunks past the end of a warp's K slice are multiplied by
// weight words that the decode kernel reads from a zero region of its own in shared memory (never
// from the ring or its padding), so their product is zero whatever the slots hold.
//
// The first call on a device looks up the array's device address (no allocation, but a
// runtime call that is not a stream operation): make that first call before any stream
// capture begins.
#include <atomic>

#include "common.cuh"

namespace bitnet {

constexpr size_t kStaticScratchBytes = 136 * 1024;

// File-scope scratch.  In host code this name is only a handle for the runtime: the device
// address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// One address per device, filled by the first call made with that device current.  Host threads
// may make that first call at the same time: they resolve the same address, and the slot is atomic.
static std::atomic<void *> g_scratch_addr[64];

static bitnet_status_t static_scratch(void **out)
{
    int dev = 0;
    BITNET_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(BITNET_ERR_DEVICE, "device index %d out of range", dev);
    void *ptr = g_scratch_addr[dev].load(std::memory_order_acquire);
    if (!ptr) {
        const cudaError_t err = cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (err != cudaSuccess || !ptr) return check_cuda(err == cudaSuccess ? cudaErrorInvalidSymbol : err, "cudaGetSymbolAddress(static scratch)");
        g_scratch_addr[dev].store(ptr, std::memory_order_release);
    }
    *out = ptr;
    return BITNET_OK;
}

}  // namespace bitnet

using namespace bitnet;

extern "C" bitnet_status_t bitnet_bitlinear_forward_static(const uint8_t *weights_dev, float w_scale, const float *x_dev,
                                                           float *y_dev, size_t M, size_t K, size_t N,
                                                           bitnet_stream_t stream)
{
    if (M == 0 || N == 0) return BITNET_OK;
    if (K == 0) return fail(BITNET_ERR_INCOMPATIBLE_SHAPES, "bitnet_bitlinear_forward_static: K == 0");
    if (!weights_dev || !x_dev || !y_dev) return fail(BITNET_ERR_NULL_POINTER, "bitnet_bitlinear_forward_static: null buffer");
    if (!decode_supports(M, K, N))
        return fail(BITNET_ERR_UNSUPPORTED_OPERATION,
                    "bitnet_bitlinear_forward_static covers the decode shapes only: 1 <= M <= 16, K %% 64 == 0, "
                    "K <= 16384 (8192 for M > 8); got M=%zu K=%zu N=%zu", M, K, N);
    const size_t need = decode_image_bytes_always(M, K, N, false);
    if (need > kStaticScratchBytes)
        return fail(BITNET_ERR_WORKSPACE, "shape needs %zu bytes of scratch, the built-in array holds %zu", need,
                    kStaticScratchBytes);
    void *scratch = nullptr;
    BITNET_TRY(static_scratch(&scratch));

    ForwardArgs a = {};
    a.wp = weights_dev; a.w_scale = w_scale; a.x = x_dev; a.y = y_dev;
    a.M = M; a.K = K; a.N = N; a.ldy = N;
    a.image_ws = scratch; a.image_ws_bytes = kStaticScratchBytes; a.force_split = true;
    return launch_decode(a, as_stream(stream));
}
