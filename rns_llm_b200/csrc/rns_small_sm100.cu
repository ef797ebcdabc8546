// Few-token RNS linear (decode steps, merged single-token requests) in ONE launch.
//
// At M <= 32 tokens the work is the stream of the 1 B/value weight matrix and a
// handful of launches' worth of latency; a 128-row tcgen05 tile would idle 7/8 of the
// tensor core and the two-launch path (quantiser, then GEMM with its tensor-memory and
// pipeline set-up) costs more in fixed latency than the arithmetic.  This kernel does
// the whole of RNSLinear.forward for such calls (src/rns_llm/layers/rns_linear.py:
// 237-275 of the reference): per-tensor or per-row absmax and quantisation of the
// activations, their residues per channel (the int8 weight serves every channel as the
// representative of its residue class), one int8 dot product per residue channel,
// mixed-radix reconstruction, dequantisation, bias, store.
//
// One CTA (4 warps) owns 8 output features and up to 16 tokens.  Every CTA quantises the
// (small) activation block itself and keeps its residues in shared memory in the
// fragment order of mma.sync.m16n8k32; the four warps split K, each requests the weight
// words of its first K steps before anything else (packed layout, straight from global
// memory, so that they arrive during the quantisation), issues one
// mma.sync.m16n8k32.s8 per channel and K step, and the partial sums meet in shared
// memory, where one thread per output reconstructs and stores.  No scratch in global
// memory, no second launch, nothing to allocate.
#include "rns_common.cuh"
#include "rns_mma_sync.cuh"

#include <cfloat>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <atomic>
#include <type_traits>

namespace rns {

constexpr int kSmallWarps = 4;
constexpr int kSmallAhead = 8;         // K steps per warp whose weight words are requested before the quantisation
constexpr int kSmallThreads = kSmallWarps * 32;
constexpr int kSmallFeatures = 8;      // output features per CTA (the n of m16n8k32)
constexpr int kSmallTokens = 16;       // tokens per CTA (the m of m16n8k32)
constexpr int kSmallMaxTokens = 32;    // absmax is recomputed by every CTA: keep the block small

struct SmallParams {
    Plan plan;
    const void* x;            // activations: floating [M,K] (quantised here) or int8 [M,K]
    int32_t x_type;           // rns_float_type, or -1 for int8 activations
    int32_t m, n, k;
    int64_t ldx;
    int32_t per_row;
    const int8_t* w;          // packed weights [K_pad/64][w_npad][64]
    int64_t w_npad;
    void* out;
    int64_t ldo;
    int32_t out_type;
    const float* col_scale;
    const float* bias;
};

template <typename T> __device__ __forceinline__ float small_load(const T* p, int64_t i);
template <> __device__ __forceinline__ float small_load<__half>(const __half* p, int64_t i) { return __half2float(p[i]); }
template <> __device__ __forceinline__ float small_load<__nv_bfloat16>(const __nv_bfloat16* p, int64_t i) { return __bfloat162float(p[i]); }
template <> __device__ __forceinline__ float small_load<float>(const float* p, int64_t i) { return p[i]; }

// Eight consecutive activations starting at element `i` (a multiple of 8) of a row with
// `valid` elements left; one 16-byte load when the address allows it.
template <typename T>
__device__ __forceinline__ void small_load8(const T* row, int i, int valid, bool vec, float (&v)[8]) {
    if (vec && valid >= 8) {
        if constexpr (sizeof(T) == 2) {
            const uint4 raw = *reinterpret_cast<const uint4*>(row + i);
            const T* h = reinterpret_cast<const T*>(&raw);
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = small_load<T>(h, j);
        } else {
            const float4 lo = *reinterpret_cast<const float4*>(row + i);
            const float4 hi = *reinterpret_cast<const float4*>(row + i + 4);
            v[0] = (float)lo.x; v[1] = (float)lo.y; v[2] = (float)lo.z; v[3] = (float)lo.w;
            v[4] = (float)hi.x; v[5] = (float)hi.y; v[6] = (float)hi.z; v[7] = (float)hi.w;
        }
    } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = j < valid ? small_load<T>(row, i + j) : 0.0f;
    }
}

template <int R, typename T>
__global__ void __launch_bounds__(kSmallThreads)
rns_linear_small_kernel(const __grid_constant__ SmallParams p) {
    extern __shared__ __align__(16) uint8_t smem[];
    __shared__ float s_part[kSmallWarps];
    __shared__ float s_row_scale[kSmallTokens];
    __shared__ int s_partial[kSmallWarps][R][kSmallTokens * kSmallFeatures];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ksteps = (p.k + 31) / 32;
    const int n0 = blockIdx.x * kSmallFeatures;
    const int m0 = blockIdx.y * kSmallTokens;
    const int rows = min(kSmallTokens, p.m - m0);
    constexpr bool kIntegers = std::is_same<T, int8_t>::value;

    // ---------------- weight words of this lane's first K steps, requested now ----------------
    // The kernel is a chain of latencies (activations, their absmax, the weights, the
    // reduction); the weight bytes do not depend on the activations, so their loads go out
    // first and land while the token block is quantised.
    const int wg = lane >> 2, wt = lane & 3;
    const int wrow = n0 + wg;                                     // weight row (output feature) of this lane
    const bool wrow_ok = wrow < p.n;
    const int wswz = (wrow >> 1) & 3;
    auto load_weight_words = [&](int s, uint32_t& w0, uint32_t& w1) {
        // bytes s*32 + 4t .. +3 and s*32 + 16 + 4t .. +3 of weight row wrow
        w0 = 0u; w1 = 0u;
        if (wrow_ok) {
            const int kb = s >> 1, base = (s & 1) * 32;
            const int8_t* rowp = p.w + ((int64_t)kb * p.w_npad + wrow) * kPackK;
            const int b0 = base + 4 * wt, b1 = base + 16 + 4 * wt;
            w0 = __ldg(reinterpret_cast<const uint32_t*>(rowp + ((((b0 >> 4) ^ wswz) << 4) | (b0 & 15))));
            w1 = __ldg(reinterpret_cast<const uint32_t*>(rowp + ((((b1 >> 4) ^ wswz) << 4) | (b1 & 15))));
        }
    };
    uint32_t ahead0[kSmallAhead], ahead1[kSmallAhead];
#pragma unroll
    for (int i = 0; i < kSmallAhead; ++i) {
        const int s = warp + i * kSmallWarps;
        ahead0[i] = 0u; ahead1[i] = 0u;
        if (s < ksteps) load_weight_words(s, ahead0[i], ahead1[i]);
    }

    // ---------------- activation scale(s) ----------------
    const int groups_per_row = (p.k + 7) / 8;                    // groups of 8 consecutive columns
    bool vec = false;
    if constexpr (!kIntegers) {
        const T* x = static_cast<const T*>(p.x);
        vec = (p.k % 8 == 0) && ((p.ldx * sizeof(T)) % 16 == 0) && (reinterpret_cast<uintptr_t>(p.x) % 16 == 0);
        if (p.per_row) {
            // one warp per row of this CTA's token block
            for (int r = warp; r < rows; r += kSmallWarps) {
                float best = 0.0f;
                const T* row = x + (int64_t)(m0 + r) * p.ldx;
                for (int gi = lane; gi < groups_per_row; gi += 32) {
                    float v[8];
                    small_load8<T>(row, gi * 8, p.k - gi * 8, vec, v);
#pragma unroll
                    for (int j = 0; j < 8; ++j) best = fmaxf(best, fabsf(v[j]));
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) best = fmaxf(best, __shfl_xor_sync(0xffffffffu, best, o));
                if (lane == 0) s_row_scale[r] = fmaxf(__fdiv_rn(best, 127.0f), FLT_EPSILON);
            }
        } else {
            // the tensor's absmax: every CTA scans all M rows (M is small)
            float best = 0.0f;
            const int total = p.m * groups_per_row;
            for (int i = threadIdx.x; i < total; i += kSmallThreads) {
                const int r = i / groups_per_row, gi = i - r * groups_per_row;
                float v[8];
                small_load8<T>(x + (int64_t)r * p.ldx, gi * 8, p.k - gi * 8, vec, v);
#pragma unroll
                for (int j = 0; j < 8; ++j) best = fmaxf(best, fabsf(v[j]));
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) best = fmaxf(best, __shfl_xor_sync(0xffffffffu, best, o));
            if (lane == 0) s_part[warp] = best;
            __syncthreads();
            if (threadIdx.x < kSmallTokens) {
                float v = fmaxf(fmaxf(s_part[0], s_part[1]), fmaxf(s_part[2], s_part[3]));
                s_row_scale[threadIdx.x] = fmaxf(__fdiv_rn(v, 127.0f), FLT_EPSILON);
            }
        }
        __syncthreads();
    }

    // ---------------- quantise + encode the token block into shared memory ----------------
    // One thread per group of eight consecutive K bytes of one row (two words of residues
    // per channel, 8 bytes apart from nothing: they are neighbours inside a 16-byte half).
    {
        const int groups_padded = ksteps * 4;                     // groups per padded row
        for (int idx = threadIdx.x; idx < kSmallTokens * groups_padded; idx += kSmallThreads) {
            const int r = idx / groups_padded;
            const int gi = idx - r * groups_padded;
            const int c0 = gi * 8;
            uint32_t word[2] = {0u, 0u};
            if (r < rows && c0 < p.k) {
                int q[8];
                if constexpr (kIntegers) {
                    const int8_t* row = static_cast<const int8_t*>(p.x) + (int64_t)(m0 + r) * p.ldx;
#pragma unroll
                    for (int j = 0; j < 8; ++j) q[j] = c0 + j < p.k ? (int)row[c0 + j] : 0;
                } else {
                    float v[8];
                    small_load8<T>(static_cast<const T*>(p.x) + (int64_t)(m0 + r) * p.ldx, c0, p.k - c0, vec, v);
                    const float scale = s_row_scale[r];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        float t = rintf(__fdiv_rn(v[j], scale));
                        q[j] = (int)fminf(fmaxf(t, -127.0f), 127.0f);
                    }
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) word[j >> 2] |= (uint32_t)(q[j] & 0xff) << (8 * (j & 3));
            }
            const int kstep = c0 >> 5, byte_in_step = c0 & 31;
#pragma unroll
            for (int c = 0; c < R; ++c) {
                uint2 e;
                e.x = encode_word_reduced(word[0] ^ 0x80808080u, fold_pattern(word[0]), p.plan.enc_mfold[c]);
                e.y = encode_word_reduced(word[1] ^ 0x80808080u, fold_pattern(word[1]), p.plan.enc_mfold[c]);
                *reinterpret_cast<uint2*>(smem + small_a_offset(c, kstep, ksteps, r, byte_in_step)) = e;
            }
        }
    }
    __syncthreads();

    // ---------------- per-channel dot products: warps split the K steps ----------------
    int acc[R][4];
#pragma unroll
    for (int c = 0; c < R; ++c) { acc[c][0] = acc[c][1] = acc[c][2] = acc[c][3] = 0; }
    {
        // One K step of one channel set.  The weight operand of EVERY channel is the int8
        // weight itself: a representative of its residue class for any modulus, so the sums
        // differ from those of canonical residues by multiples of the modulus only, and
        // |a_c| <= 128, |w| <= 128 keep them far inside int32 at the K this kernel takes.
        auto step = [&](int s, uint32_t w0, uint32_t w1) {
            const uint32_t b[2] = {w0, w1};
#pragma unroll
            for (int c = 0; c < R; ++c) {
                uint32_t a[4];
                const uint8_t* ap = smem + small_a_offset(c, s, ksteps, 0, 0);
                a[0] = *reinterpret_cast<const uint32_t*>(ap + wg * 16 + 4 * wt);
                a[1] = *reinterpret_cast<const uint32_t*>(ap + (wg + 8) * 16 + 4 * wt);
                a[2] = *reinterpret_cast<const uint32_t*>(ap + 256 + wg * 16 + 4 * wt);
                a[3] = *reinterpret_cast<const uint32_t*>(ap + 256 + (wg + 8) * 16 + 4 * wt);
                mma_s8(acc[c], a, b);
            }
        };
#pragma unroll
        for (int i = 0; i < kSmallAhead; ++i) {
            const int s = warp + i * kSmallWarps;
            if (s < ksteps) step(s, ahead0[i], ahead1[i]);
        }
        for (int s = warp + kSmallAhead * kSmallWarps; s < ksteps; s += kSmallWarps) {
            uint32_t w0, w1;
            load_weight_words(s, w0, w1);
            step(s, w0, w1);
        }
        const int g = wg, t = wt;
        // fragment -> [token][feature]: c0,c1 = row g, features 2t, 2t+1; c2,c3 = row g + 8
#pragma unroll
        for (int c = 0; c < R; ++c) {
            s_partial[warp][c][g * kSmallFeatures + 2 * t] = acc[c][0];
            s_partial[warp][c][g * kSmallFeatures + 2 * t + 1] = acc[c][1];
            s_partial[warp][c][(g + 8) * kSmallFeatures + 2 * t] = acc[c][2];
            s_partial[warp][c][(g + 8) * kSmallFeatures + 2 * t + 1] = acc[c][3];
        }
    }
    __syncthreads();

    // ---------------- reconstruction and store: one thread per output ----------------
    {
        const int r = threadIdx.x >> 3, f = threadIdx.x & 7;     // 16 tokens x 8 features = 128 threads
        const int tok = m0 + r, feat = n0 + f;
        if (r < rows && feat < p.n) {
            int sums[R];
#pragma unroll
            for (int c = 0; c < R; ++c)
                sums[c] = s_partial[0][c][threadIdx.x] + s_partial[1][c][threadIdx.x] +
                          s_partial[2][c][threadIdx.x] + s_partial[3][c][threadIdx.x];
            const long long xv = reconstruct<R>(sums, p.plan, R);
            const int64_t o = (int64_t)tok * p.ldo + feat;
            if (p.out_type == RNS_OUT_INT64) {
                static_cast<long long*>(p.out)[o] = xv;
            } else if (p.out_type == RNS_OUT_INT32) {
                static_cast<int*>(p.out)[o] = (int)xv;
            } else {
                float xf;
                if constexpr (R <= 4) xf = __int2float_rn((int)xv);
                else xf = __ll2float_rn(xv);
                float y = __fmul_rn(__fmul_rn(xf, kIntegers ? 1.0f : s_row_scale[r]), p.col_scale[feat]);
                if (p.bias != nullptr) y = __fadd_rn(y, p.bias[feat]);
                if (p.out_type == RNS_OUT_F16) static_cast<__half*>(p.out)[o] = __float2half_rn(y);
                else if (p.out_type == RNS_OUT_BF16) static_cast<__nv_bfloat16*>(p.out)[o] = __float2bfloat16_rn(y);
                else static_cast<float*>(p.out)[o] = y;
            }
        }
    }
}

template <int R, typename T>
static int launch_small(const SmallParams& sp, size_t smem_bytes, cudaStream_t st) {
    static std::atomic<uint64_t> configured{0};
    int dev = 0;
    RNS_CUDA_OK(cudaGetDevice(&dev));
    const uint64_t bit = 1ull << (dev & 63);
    // static + dynamic shared memory can pass the 48 KB default: opt in once per device
    if (!(configured.load(std::memory_order_acquire) & bit)) {
        RNS_CUDA_OK(cudaFuncSetAttribute(rns_linear_small_kernel<R, T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         96 * 1024));
        configured.fetch_or(bit, std::memory_order_release);
    }
    const dim3 grid((unsigned)((sp.n + kSmallFeatures - 1) / kSmallFeatures),
                    (unsigned)((sp.m + kSmallTokens - 1) / kSmallTokens), 1);
    rns_linear_small_kernel<R, T><<<grid, kSmallThreads, smem_bytes, st>>>(sp);
    RNS_CUDA_OK(cudaGetLastError());
    return RNS_OK;
}

template <typename T>
static int dispatch_small(const SmallParams& sp, size_t smem_bytes, cudaStream_t st) {
    switch (sp.plan.channels) {
        case 2: return launch_small<2, T>(sp, smem_bytes, st);
        case 3: return launch_small<3, T>(sp, smem_bytes, st);
        case 4: return launch_small<4, T>(sp, smem_bytes, st);
        case 5: return launch_small<5, T>(sp, smem_bytes, st);
        case 6: return launch_small<6, T>(sp, smem_bytes, st);
        default: return fail(RNS_ERR_UNSUPPORTED, "rns_linear_small covers 2..6 channels");
    }
}

static size_t small_smem_bytes(int k, int channels) { return (size_t)channels * ((k + 31) / 32) * 512; }

}  // namespace rns

using namespace rns;

extern "C" {

int rns_linear_small_supported(int m, int k, int channels) {
    return m >= 1 && m <= kSmallMaxTokens && k >= 16 && k % 16 == 0 && channels >= 2 && channels <= 6 &&
           small_smem_bytes(k, channels) <= 96 * 1024 && (int64_t)k * 128 * 128 <= (int64_t)INT32_MAX;
}

int rns_linear_small(const void* d_x, int x_type, int m, int k, int64_t ldx, int per_row,
                     const int8_t* d_w_packed, int n, const int32_t* moduli, int channels,
                     const float* d_col_scale, const float* d_bias, void* d_out, int64_t ldo,
                     int32_t out_type, rns_stream_t stream) {
    SmallParams sp;
    memset(&sp, 0, sizeof(sp));
    if (!moduli) return fail(RNS_ERR_INVALID_ARGUMENT, "rns_linear_small: moduli is NULL");
    if (int rc = build_plan(moduli, channels, &sp.plan)) return rc;
    if (!d_x || !d_w_packed || !d_out) return fail(RNS_ERR_INVALID_ARGUMENT, "rns_linear_small: NULL pointer");
    if (m <= 0 || n <= 0 || k <= 0 || ldx < k || ldo < n)
        return fail(RNS_ERR_INVALID_ARGUMENT, "rns_linear_small: bad shape or stride");
    if (!rns_linear_small_supported(m, k, channels))
        return fail(RNS_ERR_UNSUPPORTED, "rns_linear_small: needs M <= %d, K %% 16 == 0, 2..6 channels and "
                                         "channels * K <= 196608 (use rns_linear_fused otherwise)", kSmallMaxTokens);
    if (out_type < RNS_OUT_INT64 || out_type > RNS_OUT_F32)
        return fail(RNS_ERR_INVALID_ARGUMENT, "rns_linear_small: unknown out_type");
    const bool is_float_out = out_type >= RNS_OUT_F16;
    if (is_float_out && !d_col_scale)
        return fail(RNS_ERR_INVALID_ARGUMENT, "rns_linear_small: floating outputs need d_col_scale");
    if (out_type == RNS_OUT_INT32 && (sp.plan.product[channels] >> 1) >= (1ll << 31))
        return fail(RNS_ERR_OVERFLOW, "int32 output needs product(moduli)/2 < 2^31");
    if (x_type == -1 && per_row)
        return fail(RNS_ERR_INVALID_ARGUMENT, "rns_linear_small: per_row applies to floating activations");
    sp.x = d_x; sp.x_type = x_type; sp.m = m; sp.n = n; sp.k = k; sp.ldx = ldx; sp.per_row = per_row ? 1 : 0;
    sp.w = d_w_packed; sp.w_npad = round_up_i64(n, kPackNPad);
    sp.out = d_out; sp.ldo = ldo; sp.out_type = out_type;
    sp.col_scale = d_col_scale; sp.bias = d_bias;
    const size_t smem = small_smem_bytes(k, channels);
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    switch (x_type) {
        case -1: return dispatch_small<int8_t>(sp, smem, st);
        case RNS_F16: return dispatch_small<__half>(sp, smem, st);
        case RNS_BF16: return dispatch_small<__nv_bfloat16>(sp, smem, st);
        case RNS_F32: return dispatch_small<float>(sp, smem, st);
        default: return fail(RNS_ERR_INVALID_ARGUMENT, "rns_linear_small: unknown activation type");
    }
}

}  // extern "C"
