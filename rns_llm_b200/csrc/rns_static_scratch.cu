// rns_linear_static: the floating-point RNS linear for callers that cannot
// allocate device memory.
//
// The ordinary path (rns_quantize_activations + rns_linear_fused) needs somewhere
// to put the quantised activations, their scale and a reduction word; the Python
// layer takes that from its per-stream arena, which is torch's allocator
// underneath.  A host that binds this library straight through the C ABI - a
// C or C++ serving loop that receives input and output buffers from its own
// framework and is not allowed to call cudaMalloc on the request path (it may
// not own an allocator at all, and cudaMalloc serialises the device) - has no
// such place.  For those callers the scratch lives in this translation unit, in
// a fixed device array that every GPU loading the library carries until the
// process exits.
#include "rns_common.cuh"

#include <atomic>
#include <mutex>

namespace {

constexpr size_t kControlBytes = 256;                        // reduction word + scale
constexpr size_t kStaticBytes = RNS_STATIC_SCRATCH_BYTES;     // packed activations
constexpr int kMaxDevices = 64;

// Device array.  In host code this name is only a handle for
// cudaGetSymbolAddress; the address kernels receive is looked up per device.
static __device__ __align__(256) unsigned char g_static_scratch[kControlBytes + kStaticBytes];

std::mutex g_setup_mutex;
std::atomic<unsigned char*> g_device_ptr[kMaxDevices];

// First call on each device (with that device current) resolves the array's
// device address.  No allocation happens here or anywhere below.  The address is
// remembered per device ordinal; cudaDeviceReset invalidates it (a process that
// resets a device must not call rns_linear_static on it again).
int scratch_for_current_device(unsigned char** out) {
    int dev = 0;
    RNS_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices)
        return rns::fail(RNS_ERR_UNSUPPORTED, "rns_linear_static supports device ordinals below %d", kMaxDevices);
    unsigned char* ptr = g_device_ptr[dev].load(std::memory_order_acquire);
    if (ptr == nullptr) {
        std::lock_guard<std::mutex> lock(g_setup_mutex);
        ptr = g_device_ptr[dev].load(std::memory_order_acquire);
        if (ptr == nullptr) {
            void* resolved = nullptr;
            RNS_CUDA_OK(cudaGetSymbolAddress(&resolved, g_static_scratch));
            ptr = static_cast<unsigned char*>(resolved);
            g_device_ptr[dev].store(ptr, std::memory_order_release);
        }
    }
    *out = ptr;
    return RNS_OK;
}

}  // namespace

extern "C" {

int64_t rns_static_scratch_bytes(void) { return (int64_t)kStaticBytes; }

int rns_linear_static(const void* d_x, rns_float_type type, int m, int k, int64_t ldx,
                      const int8_t* d_w_packed, int n, const int32_t* moduli, int channels,
                      const float* d_col_scale, const float* d_bias, void* d_out, int64_t ldo,
                      int32_t out_type, int32_t* d_status, rns_stream_t stream) {
    // Everything is checked before the first launch: a refused call queues nothing
    // and leaves the shared array as the previous call left it.
    if (!d_x || !d_w_packed || !d_col_scale || !d_out || !moduli)
        return rns::fail(RNS_ERR_INVALID_ARGUMENT, "rns_linear_static: NULL pointer");
    if (out_type != RNS_OUT_F16 && out_type != RNS_OUT_BF16 && out_type != RNS_OUT_F32)
        return rns::fail(RNS_ERR_INVALID_ARGUMENT, "rns_linear_static produces floating outputs only");
    if (type != RNS_F16 && type != RNS_BF16 && type != RNS_F32)
        return rns::fail(RNS_ERR_INVALID_ARGUMENT, "rns_linear_static: unknown float type");
    if (m <= 0 || n <= 0 || k <= 0 || ldx < k || ldo < n)
        return rns::fail(RNS_ERR_INVALID_ARGUMENT, "rns_linear_static: bad shape or stride");
    if (channels < 2 || channels > RNS_TC_MAX_CHANNELS || !rns_linear_fused_supported(moduli, channels, k, 16, 16))
        return rns::fail(RNS_ERR_UNSUPPORTED,
                         "rns_linear_static: needs K %% 16 == 0 and 2..%d pairwise coprime moduli in [2,255]",
                         RNS_TC_MAX_CHANNELS);
    if ((int64_t)k * 128 * 128 > (int64_t)INT32_MAX)
        return rns::fail(RNS_ERR_OVERFLOW, "rns_linear_static: K = %d overflows the int32 channel sums", k);
    const int64_t need = rns_packed_activation_bytes(m, k, 1);
    if (need <= 0) return rns::fail(RNS_ERR_INVALID_ARGUMENT, "rns_linear_static: bad shape");
    if ((size_t)need > kStaticBytes)
        return rns::fail(RNS_ERR_UNSUPPORTED,
                         "rns_linear_static: %d x %d activations need %lld bytes of scratch, the built-in "
                         "array holds %lld; use rns_quantize_activations + rns_linear_fused with your own scratch",
                         m, k, (long long)need, (long long)kStaticBytes);
    unsigned char* scratch = nullptr;
    if (int rc = scratch_for_current_device(&scratch)) return rc;
    // Control block: [0,16) reduction word of the quantiser (it clears the word
    // itself on the stream before use), [64,68) the activation scale.
    void* reduction = scratch;
    float* scale = reinterpret_cast<float*>(scratch + 64);
    int8_t* packed = reinterpret_cast<int8_t*>(scratch + kControlBytes);
    if (int rc = rns_quantize_activations(d_x, type, m, k, ldx, 0, 0, /*per_row=*/0, 127, moduli, channels,
                                          packed, nullptr, /*packed_out=*/1, scale, nullptr, reduction, stream))
        return rc;
    rns_linear_args args;
    memset(&args, 0, sizeof(args));
    args.m = m; args.n = n; args.k = k;
    args.channels = channels;
    for (int i = 0; i < channels && i < RNS_MAX_CHANNELS; ++i) args.moduli[i] = moduli[i];
    args.d_a = packed;
    args.lda = k;
    args.a_packed = 1;
    args.d_w = d_w_packed;
    args.ldw = k;
    args.w_packed = 1;
    args.d_out = d_out;
    args.ldo = ldo;
    args.out_type = out_type;
    args.d_row_scale = scale;
    args.row_scale_stride = 0;
    args.d_col_scale = d_col_scale;
    args.d_bias = d_bias;
    args.d_status = d_status;
    args.pair_mode = 2;
    return rns_linear_fused(&args, stream);
}

}  // extern "C"
