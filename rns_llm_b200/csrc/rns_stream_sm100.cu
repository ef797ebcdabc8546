// Few-token RNS linear on LARGE weights (decode steps of a big model: M <= 64 tokens,
// K in the thousands): the cost is the stream of the 1 B/value weight matrix, K * N bytes,
// and the kernel is built around keeping that stream in flight.
//
// rns_small_sm100.cu holds the residues of ALL K columns of a token block in shared memory
// and lets every CTA quantise the activations itself; that stops at K = 1536 (four
// channels) and repeats the quantisation N / 8 times.  Here the activations arrive
// quantised (int8 [M,K], from rns_quantize_activations, with their scale(s) on the device)
// and a CTA walks K in chunks of 512 columns:
//   - 4 warps; the CTA owns 16 tokens x 32 output features, warp w the 8 features
//     n0 + 8w .. + 7 (one n-tile of mma.sync.m16n8k32), for ALL of K: no partial sums meet;
//   - per chunk all threads form the residues of the 16 x 512 int8 activations (one fold
//     pattern per word, a multiply-add and an xor per channel) in shared memory, fragment-major
//     (a lane's four A words side by side: one 128-bit load per fragment); then every warp runs
//     the chunk's 16 K steps: one mma per channel and step, the B fragment = the int8 weight
//     words themselves (every channel's operand, as in the other kernels);
//   - a lane keeps the weight words of 16 K steps in registers, requested one chunk ahead
//     (2 words per step): 4 KB per warp in flight, about 40 KB per SM with three CTAs
//     resident - the latency-bandwidth product of HBM.
// Epilogue per lane: its 4 outputs (tokens g, g + 8; features 2t, 2t + 1) are reconstructed,
// scaled and stored (two-byte outputs as feature pairs).
#include "rns_common.cuh"
#include "rns_mma_sync.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <atomic>

namespace rns {

constexpr int kStreamWarps = 4;
constexpr int kStreamThreads = kStreamWarps * 32;
constexpr int kStreamFeatures = 8 * kStreamWarps;   // output features per CTA
constexpr int kStreamTokens = 16;
constexpr int kStreamChunk = 512;                    // K columns per chunk
constexpr int kStreamSteps = kStreamChunk / 32;      // K steps of 32 bytes per chunk
constexpr int kStreamMaxTokens = 64;

struct StreamParams {
    Plan plan;
    const int8_t* q;          // quantised activations [M,K]
    int64_t ldq;
    int32_t m, n, k;
    const int8_t* w;          // packed weights [K_pad/64][w_npad][64]
    int64_t w_npad;
    void* out;
    int64_t ldo;
    int32_t out_type;
    const float* row_scale;   // NULL for integer outputs
    int32_t row_scale_stride; // 0: one scale, 1: per token
    const float* col_scale;
    const float* bias;
};

template <int R>
__global__ void __launch_bounds__(kStreamThreads)
rns_linear_stream_kernel(const __grid_constant__ StreamParams p) {
    // residues of one chunk: [channel][K step][lane of the mma][its four A words]
    __shared__ __align__(16) uint8_t s_a[R * kStreamSteps * 512];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int m0 = blockIdx.y * kStreamTokens;
    const int rows = min(kStreamTokens, p.m - m0);
    const int wrow = blockIdx.x * kStreamFeatures + warp * 8 + g;   // weight row of this lane (< w_npad: N_pad % 32 == 0)
    const int swz = (wrow >> 1) & 3;
    const int ksteps = (p.k + 31) / 32;                              // steps that hold data
    const int chunks = (ksteps + kStreamSteps - 1) / kStreamSteps;

    // weight words of K step s (bytes s*32 + 4t .. +3 and s*32 + 16 + 4t .. +3 of row wrow)
    auto load_weight = [&](int s, uint32_t& w0, uint32_t& w1) {
        w0 = 0u; w1 = 0u;
        if (s < ksteps) {
            const int kb = s >> 1, base = (s & 1) * 32;
            const int8_t* rowp = p.w + ((int64_t)kb * p.w_npad + wrow) * kPackK;
            const int b0 = base + 4 * t, b1 = base + 16 + 4 * t;
            w0 = __ldg(reinterpret_cast<const uint32_t*>(rowp + ((((b0 >> 4) ^ swz) << 4) | (b0 & 15))));
            w1 = __ldg(reinterpret_cast<const uint32_t*>(rowp + ((((b1 >> 4) ^ swz) << 4) | (b1 & 15))));
        }
    };
    uint32_t w0[kStreamSteps], w1[kStreamSteps];
#pragma unroll
    for (int i = 0; i < kStreamSteps; ++i) load_weight(i, w0[i], w1[i]);

    int acc[R][4];
#pragma unroll
    for (int c = 0; c < R; ++c) { acc[c][0] = acc[c][1] = acc[c][2] = acc[c][3] = 0; }

    for (int chunk = 0; chunk < chunks; ++chunk) {
        const int c0 = chunk * kStreamChunk;
        // ---- residues of this chunk's activations: one thread per 8 columns of one row ----
        for (int idx = threadIdx.x; idx < kStreamTokens * (kStreamChunk / 8); idx += kStreamThreads) {
            const int r = idx / (kStreamChunk / 8);
            const int col = (idx - r * (kStreamChunk / 8)) * 8;      // inside the chunk
            uint32_t word[2] = {0u, 0u};
            if (r < rows && c0 + col < p.k) {                        // K % 16 == 0: a group of 8 is whole
                const uint2 raw = *reinterpret_cast<const uint2*>(p.q + (int64_t)(m0 + r) * p.ldq + c0 + col);
                word[0] = raw.x; word[1] = raw.y;
            }
            // Fragment-major layout: per channel and K step, lane (g, t) of the mma owns 16
            // contiguous bytes = its four A words {row g half 0, row g+8 half 0, row g half 1,
            // row g+8 half 1}, so a fragment is ONE 128-bit shared-memory load.  The 8 columns of
            // this thread are words t0 and t0 + 1 of row r in one half of the step.
            const int kstep = col >> 5, half = (col >> 4) & 1, t0 = (col & 15) >> 2;
            const int slot = half * 2 + (r >> 3);
#pragma unroll
            for (int c = 0; c < R; ++c) {
                const uint32_t e0 = encode_word_reduced(word[0] ^ 0x80808080u, fold_pattern(word[0]), p.plan.enc_mfold[c]);
                const uint32_t e1 = encode_word_reduced(word[1] ^ 0x80808080u, fold_pattern(word[1]), p.plan.enc_mfold[c]);
                uint8_t* base = s_a + (size_t)(c * kStreamSteps + kstep) * 512 + slot * 4;
                *reinterpret_cast<uint32_t*>(base + ((r & 7) * 4 + t0) * 16) = e0;
                *reinterpret_cast<uint32_t*>(base + ((r & 7) * 4 + t0 + 1) * 16) = e1;
            }
        }
        __syncthreads();
        // ---- the chunk's K steps; the next chunk's weight words are requested as slots free ----
#pragma unroll
        for (int i = 0; i < kStreamSteps; ++i) {
            const uint32_t b[2] = {w0[i], w1[i]};
            load_weight((chunk + 1) * kStreamSteps + i, w0[i], w1[i]);
#pragma unroll
            for (int c = 0; c < R; ++c) {
                const uint4 f = *reinterpret_cast<const uint4*>(s_a + (size_t)(c * kStreamSteps + i) * 512 + lane * 16);
                const uint32_t a[4] = {f.x, f.y, f.z, f.w};
                mma_s8(acc[c], a, b);
            }
        }
        __syncthreads();                                             // before the next chunk overwrites s_a
    }

    // ---- reconstruction and store: c0,c1 = token g, features 2t, 2t+1; c2,c3 = token g + 8 ----
    const int feat0 = blockIdx.x * kStreamFeatures + warp * 8 + 2 * t;
    const bool is_float = p.out_type >= RNS_OUT_F16;
    float cs[2] = {0.0f, 0.0f}, bs[2] = {0.0f, 0.0f};
    if (is_float) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            if (feat0 + j < p.n) {
                cs[j] = p.col_scale[feat0 + j];
                if (p.bias != nullptr) bs[j] = p.bias[feat0 + j];
            }
        }
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = g + 8 * half;
        if (r >= rows) continue;
        const int tok = m0 + r;
        long long xv[2];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            int sums[R];
#pragma unroll
            for (int c = 0; c < R; ++c) sums[c] = acc[c][2 * half + j];
            xv[j] = reconstruct<R>(sums, p.plan, R);
        }
        const int64_t o = (int64_t)tok * p.ldo + feat0;
        if (!is_float) {
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                if (feat0 + j >= p.n) continue;
                if (p.out_type == RNS_OUT_INT64) static_cast<long long*>(p.out)[o + j] = xv[j];
                else static_cast<int*>(p.out)[o + j] = (int)xv[j];
            }
            continue;
        }
        const float rs = p.row_scale[p.row_scale_stride == 0 ? 0 : tok];
        float y[2];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            float xf;
            if constexpr (R <= 4) xf = __int2float_rn((int)xv[j]);
            else xf = __ll2float_rn(xv[j]);
            y[j] = __fmul_rn(__fmul_rn(xf, rs), cs[j]);
            if (p.bias != nullptr) y[j] = __fadd_rn(y[j], bs[j]);
        }
        if (p.out_type == RNS_OUT_F32) {
#pragma unroll
            for (int j = 0; j < 2; ++j)
                if (feat0 + j < p.n) static_cast<float*>(p.out)[o + j] = y[j];
            continue;
        }
        unsigned short h[2];
#pragma unroll
        for (int j = 0; j < 2; ++j)
            h[j] = p.out_type == RNS_OUT_F16 ? __half_as_ushort(__float2half_rn(y[j]))
                                             : __bfloat16_as_ushort(__float2bfloat16_rn(y[j]));
        unsigned short* out16 = static_cast<unsigned short*>(p.out);
        if (feat0 + 1 < p.n && ((o & 1) == 0) && (reinterpret_cast<uintptr_t>(p.out) & 3) == 0) {
            *reinterpret_cast<uint32_t*>(out16 + o) = (uint32_t)h[0] | ((uint32_t)h[1] << 16);
        } else {
#pragma unroll
            for (int j = 0; j < 2; ++j)
                if (feat0 + j < p.n) out16[o + j] = h[j];
        }
    }
}

template <int R>
static int launch_stream(const StreamParams& sp, cudaStream_t st) {
    const dim3 grid((unsigned)((sp.n + kStreamFeatures - 1) / kStreamFeatures),
                    (unsigned)((sp.m + kStreamTokens - 1) / kStreamTokens), 1);
    rns_linear_stream_kernel<R><<<grid, kStreamThreads, 0, st>>>(sp);
    RNS_CUDA_OK(cudaGetLastError());
    return RNS_OK;
}

}  // namespace rns

using namespace rns;

extern "C" {

int rns_linear_stream_supported(int m, int k, int channels) {
    // R * 16 K steps * 512 bytes of static shared memory must stay below the 48 KB default: R <= 5
    return m >= 1 && m <= kStreamMaxTokens && k >= 16 && k % 16 == 0 && channels >= 2 && channels <= 5 &&
           (int64_t)k * 128 * 128 <= (int64_t)INT32_MAX;
}

int rns_linear_stream(const int8_t* d_q, int m, int k, int64_t ldq, const float* d_row_scale,
                      int row_scale_stride, const int8_t* d_w_packed, int n, const int32_t* moduli,
                      int channels, const float* d_col_scale, const float* d_bias, void* d_out, int64_t ldo,
                      int32_t out_type, rns_stream_t stream) {
    StreamParams sp;
    memset(&sp, 0, sizeof(sp));
    if (!moduli) return fail(RNS_ERR_INVALID_ARGUMENT, "rns_linear_stream: moduli is NULL");
    if (int rc = build_plan(moduli, channels, &sp.plan)) return rc;
    if (!d_q || !d_w_packed || !d_out) return fail(RNS_ERR_INVALID_ARGUMENT, "rns_linear_stream: NULL pointer");
    if (m <= 0 || n <= 0 || k <= 0 || ldq < k || ldo < n)
        return fail(RNS_ERR_INVALID_ARGUMENT, "rns_linear_stream: bad shape or stride");
    if (!rns_linear_stream_supported(m, k, channels))
        return fail(RNS_ERR_UNSUPPORTED, "rns_linear_stream: needs M <= %d, K %% 16 == 0, K <= 131071 and 2..5 channels",
                    kStreamMaxTokens);
    if ((reinterpret_cast<uintptr_t>(d_q) & 7) || (ldq & 7))
        return fail(RNS_ERR_UNSUPPORTED, "rns_linear_stream: activations must be 8-byte aligned with ldq %% 8 == 0");
    if (out_type < RNS_OUT_INT64 || out_type > RNS_OUT_F32)
        return fail(RNS_ERR_INVALID_ARGUMENT, "rns_linear_stream: unknown out_type");
    const bool is_float_out = out_type >= RNS_OUT_F16;
    if (is_float_out && (!d_col_scale || !d_row_scale))
        return fail(RNS_ERR_INVALID_ARGUMENT, "rns_linear_stream: floating outputs need d_row_scale and d_col_scale");
    if (is_float_out && row_scale_stride != 0 && row_scale_stride != 1)
        return fail(RNS_ERR_INVALID_ARGUMENT, "rns_linear_stream: row_scale_stride must be 0 or 1");
    if (out_type == RNS_OUT_INT32 && (sp.plan.product[channels] >> 1) >= (1ll << 31))
        return fail(RNS_ERR_OVERFLOW, "int32 output needs product(moduli)/2 < 2^31");
    sp.q = d_q; sp.ldq = ldq; sp.m = m; sp.n = n; sp.k = k;
    sp.w = d_w_packed; sp.w_npad = round_up_i64(n, kPackNPad);
    sp.out = d_out; sp.ldo = ldo; sp.out_type = out_type;
    sp.row_scale = d_row_scale; sp.row_scale_stride = row_scale_stride;
    sp.col_scale = d_col_scale; sp.bias = d_bias;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    switch (channels) {
        case 2: return launch_stream<2>(sp, st);
        case 3: return launch_stream<3>(sp, st);
        case 4: return launch_stream<4>(sp, st);
        case 5: return launch_stream<5>(sp, st);
        default: return fail(RNS_ERR_UNSUPPORTED, "rns_linear_stream covers 2..5 channels");
    }
}

}  // extern "C"
