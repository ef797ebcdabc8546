// Plane-level kernels (the surface of the reference's FFI module) and the
// quantisation / channel-selection prologues of the fused path.  These are
// HBM-bound or tiny; the tensor-core GEMM lives in rns_gemm_sm100.cu.
#include "rns_common.cuh"

#include <cfloat>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace rns {

static inline cudaStream_t as_stream(rns_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }

static int grid_for(int64_t work, int threads, int cap = 148 * 16) {
    int64_t blocks = (work + threads - 1) / threads;
    if (blocks < 1) blocks = 1;
    if (blocks > cap) blocks = cap;
    return (int)blocks;
}

struct ModList {
    int32_t channels;
    int32_t mod[kMaxCh];
};

static ModList modlist(const Plan& p) {
    ModList l;
    l.channels = p.channels;
    for (int i = 0; i < kMaxCh; ++i) l.mod[i] = p.mod[i];
    return l;
}

// ---------------------------------------------------------------------------
// Encoders.  One thread per source element, all channels: the source is read
// once (the reference reads it once per channel, csrc/rns_cuda.cu:98-124).
// ---------------------------------------------------------------------------
template <typename T>
__global__ void encode_centered_kernel(const T* __restrict__ values, int8_t* __restrict__ out,
                                       ModList ml, int64_t elements) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < elements;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int v = (int)values[i];
#pragma unroll 1
        for (int c = 0; c < ml.channels; ++c) {
            const int m = ml.mod[c];
            int r = v % m;  // C remainder: sign of the dividend
            const int half = m / 2;
            if (r > half) r -= m;
            else if (r < -half) r += m;
            out[(int64_t)c * elements + i] = (int8_t)r;
        }
    }
}

__global__ void encode_canonical_kernel(const int8_t* __restrict__ values, uint8_t* __restrict__ out,
                                        ModList ml, int64_t elements) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < elements;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int v = (int)values[i];
#pragma unroll 1
        for (int c = 0; c < ml.channels; ++c) {
            const int m = ml.mod[c];
            int r = v % m;
            if (r < 0) r += m;
            out[(int64_t)c * elements + i] = (uint8_t)r;
        }
    }
}

// ---------------------------------------------------------------------------
// Plane GEMM: exact per-channel product of byte planes with int64 sums, tiled
// through shared memory.  Serves the plane-level entry points only (arbitrary
// shapes, B stored [K,N]); the product path is the tcgen05 kernel.
//   MODE 0: canonical uint8 in, canonical uint8 out
//   MODE 1: centred int8 in, centred int8 out
//   MODE 2: centred int8 in, raw int32 sums out
// ---------------------------------------------------------------------------
constexpr int kPT = 32;  // output tile edge
constexpr int kPK = 32;  // k slab

template <int MODE>
__global__ void __launch_bounds__(256)
plane_gemm_kernel(const void* __restrict__ a_, const void* __restrict__ b_, void* __restrict__ out_,
                  ModList ml, int m, int k, int n) {
    using In = typename std::conditional<MODE == 0, uint8_t, int8_t>::type;
    const In* a = static_cast<const In*>(a_) + (int64_t)blockIdx.z * m * k;
    const In* b = static_cast<const In*>(b_) + (int64_t)blockIdx.z * k * n;
    __shared__ int sa[kPT][kPK + 1];
    __shared__ int sb[kPK][kPT + 1];
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;  // each thread: 2x2 outputs
    const int row0 = blockIdx.y * kPT, col0 = blockIdx.x * kPT;
    long long acc[2][2] = {{0, 0}, {0, 0}};
    for (int k0 = 0; k0 < k; k0 += kPK) {
        for (int idx = threadIdx.x; idx < kPT * kPK; idx += 256) {
            const int r = idx / kPK, c = idx % kPK;
            const int gr = row0 + r, gc = k0 + c;
            sa[r][c] = (gr < m && gc < k) ? (int)a[(int64_t)gr * k + gc] : 0;
            const int br = idx / kPT, bc = idx % kPT;
            const int gbr = k0 + br, gbc = col0 + bc;
            sb[br][bc] = (gbr < k && gbc < n) ? (int)b[(int64_t)gbr * n + gbc] : 0;
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < kPK; ++kk) {
            const int a0 = sa[ty * 2][kk], a1 = sa[ty * 2 + 1][kk];
            const int b0 = sb[kk][tx * 2], b1 = sb[kk][tx * 2 + 1];
            acc[0][0] += a0 * b0; acc[0][1] += a0 * b1;
            acc[1][0] += a1 * b0; acc[1][1] += a1 * b1;
        }
        __syncthreads();
    }
    const int mod = ml.mod[blockIdx.z];
    for (int i = 0; i < 2; ++i)
        for (int j = 0; j < 2; ++j) {
            const int gr = row0 + ty * 2 + i, gc = col0 + tx * 2 + j;
            if (gr >= m || gc >= n) continue;
            const int64_t o = ((int64_t)blockIdx.z * m + gr) * n + gc;
            if (MODE == 2) {
                static_cast<int32_t*>(out_)[o] = (int32_t)acc[i][j];
            } else {
                long long r = acc[i][j] % mod;
                if (MODE == 0) {
                    if (r < 0) r += mod;
                    static_cast<uint8_t*>(out_)[o] = (uint8_t)r;
                } else {
                    const int half = mod / 2;
                    if (r > half) r -= mod;
                    else if (r < -half) r += mod;
                    static_cast<int8_t*>(out_)[o] = (int8_t)r;
                }
            }
        }
}

// ---------------------------------------------------------------------------
// Reconstruction from planes: SRC = int8 centred residues or int32 raw sums.
// ---------------------------------------------------------------------------
template <int R, typename SRC>
__global__ void __launch_bounds__(256)
garner_planes_kernel(const SRC* __restrict__ src, int64_t* __restrict__ out,
                     const __grid_constant__ Plan pl, int64_t elements) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < elements;
         i += (int64_t)gridDim.x * blockDim.x) {
        int acc[R];
#pragma unroll
        for (int c = 0; c < R; ++c) acc[c] = (int)src[(int64_t)c * elements + i];
        out[i] = reconstruct<R>(acc, pl, R);
    }
}

template <typename SRC>
static int launch_garner(const SRC* src, int64_t* out, const Plan& pl, int64_t elements,
                         cudaStream_t st) {
    const int blocks = grid_for(elements, 256);
#define RNS_CASE(RR) \
    case RR: garner_planes_kernel<RR, SRC><<<blocks, 256, 0, st>>>(src, out, pl, elements); break;
    switch (pl.channels) {
        RNS_CASE(2) RNS_CASE(3) RNS_CASE(4) RNS_CASE(5) RNS_CASE(6)
        RNS_CASE(7) RNS_CASE(8) RNS_CASE(9) RNS_CASE(10)
        default:
            return fail(RNS_ERR_UNSUPPORTED, "Garner reconstruction supports 2..10 channels");
    }
#undef RNS_CASE
    RNS_CUDA_OK(cudaGetLastError());
    return RNS_OK;
}

// ---------------------------------------------------------------------------
// Activation quantiser
// ---------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float load_f(const T* p, int64_t i);
template <> __device__ __forceinline__ float load_f<__half>(const __half* p, int64_t i) { return __half2float(p[i]); }
template <> __device__ __forceinline__ float load_f<__nv_bfloat16>(const __nv_bfloat16* p, int64_t i) { return __bfloat162float(p[i]); }
template <> __device__ __forceinline__ float load_f<float>(const float* p, int64_t i) { return p[i]; }

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ int warp_sum(int v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// ---------------------------------------------------------------------------
// Activation source view.  Element (r, c) of the logical [M,K] matrix lives at
//   x[(c / col_block) * col_block_stride + r * ldx + (c % col_block)]
// which covers a plain strided matrix (col_block = K) and the layout an
// all-gather of column shards leaves behind: G blocks [M, K/G] one after the
// other (col_block = K/G, col_block_stride = M*K/G, ldx = K/G).
// ---------------------------------------------------------------------------
struct SrcView {
    const void* x;
    int32_t m, k;
    int64_t ldx;
    int32_t col_block;
    int64_t col_block_stride;
    int32_t vec8;  // 1: every group of 8 columns is contiguous and 16-byte aligned
};

__device__ __forceinline__ int64_t src_offset(const SrcView& s, int r, int c) {
    if (s.col_block == s.k) return (int64_t)r * s.ldx + c;   // plain matrix: no column blocks
    const int b = c / s.col_block;
    return (int64_t)b * s.col_block_stride + (int64_t)r * s.ldx + (c - b * s.col_block);
}

// Eight consecutive columns starting at column c (a multiple of 8) of row r.
template <typename T>
__device__ __forceinline__ void load8(const SrcView& s, int r, int c, float (&v)[8]) {
    const T* base = static_cast<const T*>(s.x) + src_offset(s, r, c);
    if (s.vec8) {
        if constexpr (sizeof(T) == 2) {
            const uint4 raw = *reinterpret_cast<const uint4*>(base);
            const T* h = reinterpret_cast<const T*>(&raw);
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = load_f<T>(h, i);
        } else {
            const float4 lo = *reinterpret_cast<const float4*>(base);
            const float4 hi = *reinterpret_cast<const float4*>(base + 4);
            v[0] = lo.x; v[1] = lo.y; v[2] = lo.z; v[3] = lo.w;
            v[4] = hi.x; v[5] = hi.y; v[6] = hi.z; v[7] = hi.w;
        }
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i)
            v[i] = (c + i < s.k) ? load_f<T>(static_cast<const T*>(s.x), src_offset(s, r, c + i)) : 0.0f;
    }
}

__device__ __forceinline__ int quantize_one(float v, float scale, int qmax) {
    // torch: clamp(round(v / scale), -qmax, qmax); round = ties to even.
    float q = rintf(__fdiv_rn(v, scale));
    q = fminf(fmaxf(q, (float)-qmax), (float)qmax);
    return (int)q;
}

// The same value with the division off the common path: t = v * (1/scale) is within
// 2 ulp of v / scale, so the two round to different integers only when a half-integer
// lies between them; only then (|t - round(t)| within 1e-4 of 0.5) the caller redoes
// the IEEE division (`doubtful`).  The rounding itself is clamp, then add 1.5 * 2^23 (round to nearest
// even in the adder): the sum's low mantissa bits are the integer, so neither a
// rounding nor a conversion instruction is issued.  |t| >= 127.5, infinities and NaN
// fail the same test (the clamped integer is far away, or the difference is NaN).
// Wider targets (qmax up to 32767): 2 ulp of t reach 0.002, so the margin widens to 0.01.
__device__ __forceinline__ int quantize_one_fast(float v, float inv_scale, int qmax, bool& doubtful) {
    const float t = __fmul_rn(v, inv_scale);
    const float magic = 12582912.0f;
    const float r = __fadd_rn(fminf(fmaxf(t, (float)-qmax), (float)qmax), magic);
    doubtful |= !(fabsf(t - __fsub_rn(r, magic)) <= (qmax <= 127 ? 0.4999f : 0.49f));
    return __float_as_int(r) - 0x4B400000;
}

__device__ __forceinline__ int centred_residue(int v, int m) {
    int r = v % m;
    const int half = m / 2;
    if (r > half) r -= m;
    else if (r < -half) r += m;
    return r;
}

struct QuantOut {
    int8_t* q;        // [M,K] or NULL
    int8_t* planes;   // [channels,M,K] or NULL
    float* scale;     // [1] or [M]
    int* row_l1_max;  // [1] or NULL
    int32_t channels;
    int32_t mod[kMaxCh];
    uint32_t enc_hi[kMaxCh], enc_lo[kMaxCh], enc_mk[kMaxCh], enc_mfold[kMaxCh];
    int32_t reduced;    // planes hold one-step reduced residues (packed planes of the quantiser)
    int32_t single_fold;
    int32_t fast;
    int32_t packed;     // outputs in the packed tile layouts
    int32_t kblocks;    // K_pad / 64 (packed only)
    int32_t tile_rows;  // token rows per packed tile (128, or 64 / 48 for the two-CTA kernel)
};

// Where a row falls in the packed layouts: its tile row and its row inside the tile
// (computed once per row: the tile height need not be a power of two).
struct RowPos {
    int32_t tile;
    int32_t inside;
};
__device__ __forceinline__ RowPos row_pos(const QuantOut& o, int r) {
    RowPos p;
    if (o.tile_rows == kPackM) { p.tile = r >> 7; p.inside = r & 127; }
    else { p.tile = r / o.tile_rows; p.inside = r - p.tile * o.tile_rows; }
    return p;
}

// Quantises columns [c, c+8) of row r, stores values and planes, returns sum |q|.
template <typename T>
__device__ __forceinline__ int quantize_loaded(const float (&v)[8], const SrcView& s, const QuantOut& o, int r, int c,
                                               float scale, int qmax, const RowPos pos) {
    int q[8];
    int l1 = 0;
    const float inv_scale = __frcp_rn(scale);
    bool redo = false;   // one branch per group: any doubtful value sends all eight through the division
#pragma unroll
    for (int i = 0; i < 8; ++i) q[i] = quantize_one_fast(v[i], inv_scale, qmax, redo);
    if (redo) {
#pragma unroll
        for (int i = 0; i < 8; ++i) q[i] = quantize_one(v[i], scale, qmax);
    }
    if (o.row_l1_max != nullptr) {   // only the adaptive path reads the row sums
#pragma unroll
        for (int i = 0; i < 8; ++i) l1 += q[i] < 0 ? -q[i] : q[i];
    }
    const bool full = c + 8 <= s.k;
    // low bytes of four ints -> one word: (q0.b0, q1.b0) and (q2.b0, q3.b0), then both pairs
    const uint32_t w0 = __byte_perm(__byte_perm((uint32_t)q[0], (uint32_t)q[1], 0x0040),
                                    __byte_perm((uint32_t)q[2], (uint32_t)q[3], 0x0040), 0x5410);
    const uint32_t w1 = __byte_perm(__byte_perm((uint32_t)q[4], (uint32_t)q[5], 0x0040),
                                    __byte_perm((uint32_t)q[6], (uint32_t)q[7], 0x0040), 0x5410);
    // Plain: byte offset r*K + c, planes M*K apart.  Packed: tile layouts, where a
    // group of 8 columns (c % 8 == 0) is half of one 16-byte chunk.
    // Packed: tile (r / 128, c / 64) of one channel (values) or of `channels` channels (planes).
    const int64_t tile = (int64_t)pos.tile * o.kblocks + (c >> 6);
    const int in_tile = packed_row_offset(pos.inside, c & 63);
    const int tile_bytes = o.tile_rows * kPackK;
    const int64_t off = o.packed ? tile * tile_bytes + in_tile : (int64_t)r * s.k + c;
    if (full && (off & 7) == 0) {
        if (o.q) *reinterpret_cast<uint2*>(o.q + off) = make_uint2(w0, w1);
        if (o.planes) {
            const int64_t plane = o.packed ? (int64_t)tile_bytes : (int64_t)s.m * s.k;
            const int64_t base = o.packed ? tile * o.channels * tile_bytes + in_tile : off;
            const uint32_t u0 = w0 ^ 0x80808080u, u1 = w1 ^ 0x80808080u;
            const uint32_t l0 = u0 & 0x7f7f7f7fu, l1w = u1 & 0x7f7f7f7fu;
            if (o.reduced) {
                // one fold pattern per word, then one multiply-add and one xor per channel
                const uint32_t d0 = fold_pattern(w0), d1 = fold_pattern(w1);
                int8_t* dst = o.planes + base;
#pragma unroll 4
                for (int ch = 0; ch < o.channels; ++ch, dst += plane)
                    *reinterpret_cast<uint2*>(dst) = make_uint2(encode_word_reduced(u0, d0, o.enc_mfold[ch]),
                                                                encode_word_reduced(u1, d1, o.enc_mfold[ch]));
            } else if (o.single_fold && o.fast) {
                // the common case (every modulus in [86, 127]) without per-channel branches
                int8_t* dst = o.planes + base;
#pragma unroll 4
                for (int ch = 0; ch < o.channels; ++ch, dst += plane)
                    *reinterpret_cast<uint2*>(dst) =
                        make_uint2(encode_word<true>(u0, l0, o.enc_hi[ch], o.enc_lo[ch], o.enc_mk[ch]),
                                   encode_word<true>(u1, l1w, o.enc_hi[ch], o.enc_lo[ch], o.enc_mk[ch]));
            } else
#pragma unroll 1
            for (int ch = 0; ch < o.channels; ++ch) {
                uint2 e;
                if (o.single_fold) {
                    e = make_uint2(encode_word<false>(u0, l0, o.enc_hi[ch], o.enc_lo[ch], o.enc_mk[ch]),
                                   encode_word<false>(u1, l1w, o.enc_hi[ch], o.enc_lo[ch], o.enc_mk[ch]));
                } else {
                    uint32_t e0 = 0, e1 = 0;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        e0 |= (uint32_t)(centred_residue(q[i], o.mod[ch]) & 0xff) << (8 * i);
                        e1 |= (uint32_t)(centred_residue(q[4 + i], o.mod[ch]) & 0xff) << (8 * i);
                    }
                    e = make_uint2(e0, e1);
                }
                *reinterpret_cast<uint2*>(o.planes + base + ch * plane) = e;
            }
        }
    } else {
        // ragged tail or unaligned output: plain layout only (the packed layout needs K % 8 == 0)
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (c + i < s.k) {
                if (o.q) o.q[off + i] = (int8_t)q[i];
                if (o.planes)
                    for (int ch = 0; ch < o.channels; ++ch)
                        o.planes[(int64_t)ch * s.m * s.k + off + i] = (int8_t)centred_residue(q[i], o.mod[ch]);
            }
        }
    }
    return l1;
}

// kQuantUnroll groups of a row per step, every load issued before the first group is processed.
#ifndef RNS_QUNROLL
#define RNS_QUNROLL 1
#endif
constexpr int kQuantUnroll = RNS_QUNROLL;
template <typename T>
__device__ __forceinline__ int quantize_row(const SrcView& s, const QuantOut& o, int row, int lane,
                                            int groups_per_row, float scale, int qmax, int first_group = 0) {
    int l1 = 0;
    const RowPos pos = row_pos(o, row);
    for (int g = first_group + lane; g < groups_per_row; g += 32 * kQuantUnroll) {
        float v[kQuantUnroll][8];
#pragma unroll
        for (int u = 0; u < kQuantUnroll; ++u)
            if (g + 32 * u < groups_per_row) load8<T>(s, row, (g + 32 * u) * 8, v[u]);
#pragma unroll
        for (int u = 0; u < kQuantUnroll; ++u)
            if (g + 32 * u < groups_per_row) l1 += quantize_loaded<T>(v[u], s, o, row, (g + 32 * u) * 8, scale, qmax, pos);
    }
    return l1;
}

template <typename T>
__device__ __forceinline__ float group_absmax(const SrcView& s, int r, int c) {
    float v[8];
    load8<T>(s, r, c, v);
    float best = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) best = fmaxf(best, fabsf(v[i]));
    return best;
}

// Pass 1 of the per-tensor quantiser: tensor-wide absmax by atomicMax on the
// float's bit pattern (order preserving for non-negative floats).  The scratch
// word is zeroed by a memset enqueued before the kernel.
template <typename T>
__global__ void __launch_bounds__(256)
absmax_kernel(const __grid_constant__ SrcView s, unsigned* __restrict__ scratch) {
    float best = 0.0f;
    const int groups_per_row = (s.k + 7) / 8;
    const int64_t total = (int64_t)s.m * groups_per_row;
    const unsigned stride = gridDim.x * blockDim.x;
    if (s.vec8 && total < (1ll << 31)) {
        // 32-bit index arithmetic and four independent 16-byte loads per thread and step
        const unsigned count = (unsigned)total, gpr = (unsigned)groups_per_row;
        for (unsigned g = blockIdx.x * blockDim.x + threadIdx.x; g < count; g += 4 * stride) {
            float part4[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const unsigned gi = g + u * stride;
                part4[u] = 0.0f;
                if (gi < count) {
                    const unsigned r = gi / gpr;
                    part4[u] = group_absmax<T>(s, (int)r, (int)(gi - r * gpr) * 8);
                }
            }
            best = fmaxf(fmaxf(best, fmaxf(part4[0], part4[1])), fmaxf(part4[2], part4[3]));
        }
    } else {
        for (int64_t g = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; g < total; g += stride) {
            const int r = (int)(g / groups_per_row);
            const int c = (int)(g - (int64_t)r * groups_per_row) * 8;
            best = fmaxf(best, group_absmax<T>(s, r, c));
        }
    }
    best = warp_max(best);
    __shared__ float part[8];
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x < 32) {
        float v = threadIdx.x < 8 ? part[threadIdx.x] : 0.0f;
        v = warp_max(v);
        if (threadIdx.x == 0) atomicMax(scratch, __float_as_uint(v));
    }
}

// Pass 2 (one warp per row segment): scale, int8 values, optional planes, row L1.
// PER_ROW: the warp first reduces its own row's absmax.  A row is one segment when
// its absmax or its L1 sum is wanted (segments = 1); otherwise rows are cut into
// `segments` pieces of `seg_groups` groups so that short and wide matrices both
// spread evenly over the SMs.
#ifndef RNS_QMINBLOCKS
#define RNS_QMINBLOCKS 4
#endif
// Tensor-wide absmax as the maximum of `parts` words `stride` words apart (bit patterns
// of non-negative floats: one word from this call's own absmax pass, or one per rank
// from the epilogues of a column-sharded previous layer).
__device__ __forceinline__ float absmax_of_parts(const unsigned* __restrict__ src, int parts, int64_t stride) {
    unsigned best = src[0];
    for (int i = 1; i < parts; ++i) best = max(best, src[(int64_t)i * stride]);
    return __uint_as_float(best);
}

template <typename T, bool PER_ROW>
__global__ void __launch_bounds__(256, RNS_QMINBLOCKS)
quantize_rows_kernel(const __grid_constant__ SrcView s, const __grid_constant__ QuantOut o,
                     int qmax, const unsigned* __restrict__ scratch, int parts, int64_t part_stride,
                     int segments, int seg_groups) {
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    const int groups_per_row = (s.k + 7) / 8;
    int worst_l1 = 0;
    if (!PER_ROW && segments > 1) {
        const float scale = fmaxf(__fdiv_rn(absmax_of_parts(scratch, parts, part_stride), (float)qmax), FLT_EPSILON);
        if (blockIdx.x == 0 && threadIdx.x == 0) o.scale[0] = scale;
        const int64_t units = (int64_t)s.m * segments;
        for (int64_t u = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; u < units; u += warps) {
            const int row = (int)(u / segments);
            const int first = (int)(u - (int64_t)row * segments) * seg_groups;
            quantize_row<T>(s, o, row, lane, min(groups_per_row, first + seg_groups), scale, qmax, first);
        }
        return;
    }
    for (int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; row < s.m; row += warps) {
        float absmax;
        if (PER_ROW) {
            float best = 0.0f;
            for (int g = lane; g < groups_per_row; g += 32) best = fmaxf(best, group_absmax<T>(s, row, g * 8));
            absmax = warp_max(best);
        } else {
            absmax = absmax_of_parts(scratch, parts, part_stride);
        }
        const float scale = fmaxf(__fdiv_rn(absmax, (float)qmax), FLT_EPSILON);
        if (lane == 0) {
            if (PER_ROW) o.scale[row] = scale;
            else if (row == 0) o.scale[0] = scale;
        }
        const int l1 = quantize_row<T>(s, o, row, lane, groups_per_row, scale, qmax);
        if (o.row_l1_max) worst_l1 = max(worst_l1, warp_sum(l1));
    }
    if (o.row_l1_max && lane == 0 && worst_l1 > 0) atomicMax(o.row_l1_max, worst_l1);
}

// Per-tensor quantiser for small activations in ONE launch of one CTA: absmax
// through shared memory, then the same per-row work.  No scratch, no memset.
template <typename T>
__global__ void __launch_bounds__(1024)
quantize_small_kernel(const __grid_constant__ SrcView s, const __grid_constant__ QuantOut o, int qmax) {
    __shared__ float part[32];
    __shared__ float s_absmax;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int groups_per_row = (s.k + 7) / 8;
    const int total = s.m * groups_per_row;
    float best = 0.0f;
    for (int g = threadIdx.x; g < total; g += blockDim.x) {
        const int r = g / groups_per_row;
        best = fmaxf(best, group_absmax<T>(s, r, (g - r * groups_per_row) * 8));
    }
    best = warp_max(best);
    if (lane == 0) part[warp] = best;
    if (threadIdx.x == 0 && o.row_l1_max) *o.row_l1_max = 0;
    __syncthreads();
    if (warp == 0) {
        float v = warp_max(part[lane]);
        if (lane == 0) s_absmax = v;
    }
    __syncthreads();
    const float scale = fmaxf(__fdiv_rn(s_absmax, (float)qmax), FLT_EPSILON);
    if (threadIdx.x == 0) o.scale[0] = scale;
    int worst_l1 = 0;
    for (int row = warp; row < s.m; row += (int)(blockDim.x >> 5)) {
        const int l1 = quantize_row<T>(s, o, row, lane, groups_per_row, scale, qmax);
        if (o.row_l1_max) worst_l1 = max(worst_l1, warp_sum(l1));
    }
    if (o.row_l1_max && lane == 0 && worst_l1 > 0) atomicMax(o.row_l1_max, worst_l1);
}

__global__ void __launch_bounds__(256)
row_l1_max_kernel(const int8_t* __restrict__ a, int m, int k, int64_t lda, int* __restrict__ out) {
    __shared__ int ipart[8];
    for (int row = blockIdx.x; row < m; row += gridDim.x) {
        int l1 = 0;
        for (int c = threadIdx.x; c < k; c += blockDim.x) {
            const int v = a[(int64_t)row * lda + c];
            l1 += v < 0 ? -v : v;
        }
        l1 = warp_sum(l1);
        if ((threadIdx.x & 31) == 0) ipart[threadIdx.x >> 5] = l1;
        __syncthreads();
        if (threadIdx.x == 0) {
            int total = 0;
            for (int w = 0; w < 8; ++w) total += ipart[w];
            atomicMax(out, total);
        }
        __syncthreads();
    }
}

struct SelectArgs {
    int32_t channels, min_channels, max_abs_weight;
    int64_t product[kMaxCh + 1];
};

__global__ void select_channels_kernel(const int* __restrict__ row_l1_max, SelectArgs sa,
                                       int* __restrict__ active, long long* __restrict__ meta,
                                       long long* __restrict__ histogram,
                                       int* __restrict__ status) {
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    const long long bound = (long long)(*row_l1_max) * sa.max_abs_weight;
    int chosen = 0;
    for (int c = sa.min_channels; c <= sa.channels; ++c)
        if (2 * bound < sa.product[c]) { chosen = c; break; }
    if (chosen == 0) {
        chosen = sa.channels;
        if (status) atomicExch(status, (int)RNS_ERR_OVERFLOW);
    }
    *active = chosen;
    if (meta) {
        meta[0] = chosen;
        meta[1] = bound;
        meta[2] = (sa.product[chosen] - 1) / 2;
    }
    if (histogram) histogram[chosen] += 1;
}

// Weight quantiser: one block per output channel (row of W).
template <typename T>
__global__ void __launch_bounds__(256)
quantize_weight_kernel(const T* __restrict__ w, int n, int k, int64_t ldw, int qmax,
                       int8_t* __restrict__ wq, float* __restrict__ scale_out,
                       int* __restrict__ max_abs) {
    __shared__ float part[8];
    __shared__ float s_scale;
    for (int row = blockIdx.x; row < n; row += gridDim.x) {
        const T* wr = w + (int64_t)row * ldw;
        float best = 0.0f;
        for (int c = threadIdx.x; c < k; c += blockDim.x) best = fmaxf(best, fabsf(load_f<T>(wr, c)));
        best = warp_max(best);
        if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = best;
        __syncthreads();
        if (threadIdx.x < 32) {
            float v = threadIdx.x < 8 ? part[threadIdx.x] : 0.0f;
            v = warp_max(v);
            if (threadIdx.x == 0) s_scale = fmaxf(__fdiv_rn(v, (float)qmax), FLT_EPSILON);
        }
        __syncthreads();
        const float scale = s_scale;
        if (threadIdx.x == 0) scale_out[row] = scale;
        int biggest = 0;
        for (int c = threadIdx.x; c < k; c += blockDim.x) {
            const int q = quantize_one(load_f<T>(wr, c), scale, qmax);
            wq[(int64_t)row * k + c] = (int8_t)q;
            biggest = max(biggest, q < 0 ? -q : q);
        }
        if (max_abs) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) biggest = max(biggest, __shfl_xor_sync(0xffffffffu, biggest, o));
            if ((threadIdx.x & 31) == 0) atomicMax(max_abs, biggest);
        }
        __syncthreads();
    }
}


// ---------------------------------------------------------------------------
// Packed tile layouts
// ---------------------------------------------------------------------------
// One thread per 16-byte chunk of the packed weight [K_pad/64][N_pad][64].
template <bool UNPACK>
__global__ void __launch_bounds__(256)
pack_weight_kernel(int8_t* __restrict__ plain, int8_t* __restrict__ packed, int n, int k, int64_t ldw,
                   int64_t n_pad, int kblocks) {
    const int64_t chunks = (int64_t)kblocks * n_pad * 4;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < chunks;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int chunk = (int)(i & 3);
        const int64_t row_id = i >> 2;
        const int row = (int)(row_id % n_pad);
        const int kb = (int)(row_id / n_pad);
        const int col = kb * kPackK + chunk * 16;
        int8_t* pk = packed + packed_weight_offset(row, col, n_pad);
        if (UNPACK) {
            if (row < n)
                for (int j = 0; j < 16 && col + j < k; ++j) plain[(int64_t)row * ldw + col + j] = pk[j];
        } else {
            uint4 v = make_uint4(0, 0, 0, 0);
            if (row < n && col < k) {
                const int8_t* src = plain + (int64_t)row * ldw + col;
                if (col + 16 <= k && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
                    v = *reinterpret_cast<const uint4*>(src);
                } else {
                    int8_t tmp[16] = {0};
                    for (int j = 0; j < 16 && col + j < k; ++j) tmp[j] = src[j];
                    v = *reinterpret_cast<const uint4*>(tmp);
                }
            }
            *reinterpret_cast<uint4*>(pk) = v;
        }
    }
}

// One thread per 16-byte chunk of the source activations; writes every channel.
__global__ void __launch_bounds__(256)
encode_planes_packed_kernel(const int8_t* __restrict__ a, int m, int k, int64_t lda, QuantOut o) {
    const int chunks_per_row = (k + 15) / 16;
    const int64_t chunks = (int64_t)m * chunks_per_row;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < chunks;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int row = (int)(i / chunks_per_row);
        const int col = (int)(i - (int64_t)row * chunks_per_row) * 16;
        const int8_t* src = a + (int64_t)row * lda + col;
        uint4 x;
        if (col + 16 <= k && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
            x = *reinterpret_cast<const uint4*>(src);
        } else {
            int8_t tmp[16] = {0};
            for (int j = 0; j < 16 && col + j < k; ++j) tmp[j] = src[j];
            x = *reinterpret_cast<const uint4*>(tmp);
        }
        const uint32_t w[4] = {x.x, x.y, x.z, x.w};
        // tile (row / tile_rows, col / 64) of `channels` channels, tile_rows x 64 bytes each
        const RowPos pos = row_pos(o, row);
        const int tile_bytes = o.tile_rows * kPackK;
        const int64_t base = ((int64_t)pos.tile * o.kblocks + (col >> 6)) * o.channels * tile_bytes +
                             packed_row_offset(pos.inside, col & 63);
#pragma unroll 1
        for (int ch = 0; ch < o.channels; ++ch) {
            uint32_t e[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t u = w[j] ^ 0x80808080u, ul = w[j] & 0x7f7f7f7fu;
                if (o.single_fold && o.fast) e[j] = encode_word<true>(u, ul, o.enc_hi[ch], o.enc_lo[ch], o.enc_mk[ch]);
                else if (o.single_fold) e[j] = encode_word<false>(u, ul, o.enc_hi[ch], o.enc_lo[ch], o.enc_mk[ch]);
                else {
                    e[j] = 0;
                    for (int b = 0; b < 4; ++b)
                        e[j] |= (uint32_t)(centred_residue((int)(int8_t)(w[j] >> (8 * b)), o.mod[ch]) & 0xff) << (8 * b);
                }
            }
            *reinterpret_cast<uint4*>(o.planes + base + (int64_t)ch * tile_bytes) =
                make_uint4(e[0], e[1], e[2], e[3]);
        }
    }
}

static int fill_encoder(QuantOut& qo, const int32_t* moduli, int channels) {
    Plan pl;
    if (int rc = build_plan(moduli, channels, &pl)) return rc;
    qo.channels = pl.channels;
    qo.single_fold = pl.encode_single_fold;
    qo.fast = pl.encode_fast;
    for (int i = 0; i < kMaxCh; ++i) {
        qo.mod[i] = pl.mod[i]; qo.enc_hi[i] = pl.enc_hi[i]; qo.enc_lo[i] = pl.enc_lo[i];
        qo.enc_mk[i] = pl.enc_mk[i]; qo.enc_mfold[i] = pl.enc_mfold[i];
    }
    return RNS_OK;
}

static int check_gemm_dims(const void* a, const void* b, const void* out, int m, int k, int n) {
    if (!a || !b || !out) return fail(RNS_ERR_INVALID_ARGUMENT, "plane GEMM: NULL pointer");
    if (m <= 0 || k <= 0 || n <= 0)
        return fail(RNS_ERR_INVALID_ARGUMENT, "matrix dimensions must be positive");
    return RNS_OK;
}

template <int MODE>
static int launch_plane_gemm(const void* a, const void* b, void* out, const Plan& pl, int m, int k,
                             int n, cudaStream_t st) {
    if (pl.channels > 65535) return fail(RNS_ERR_INVALID_ARGUMENT, "too many residue channels");
    dim3 grid((n + kPT - 1) / kPT, (m + kPT - 1) / kPT, pl.channels);
    plane_gemm_kernel<MODE><<<grid, 256, 0, st>>>(a, b, out, modlist(pl), m, k, n);
    RNS_CUDA_OK(cudaGetLastError());
    return RNS_OK;
}

}  // namespace rns

// ===========================================================================
// C ABI
// ===========================================================================
using namespace rns;

extern "C" {

int rns_encode_canonical_i8(const int8_t* d_values, int64_t elements, const int32_t* moduli,
                            int channels, uint8_t* d_out, rns_stream_t stream) {
    Plan pl;
    if (int rc = build_plan(moduli, channels, &pl)) return rc;
    if (elements < 0 || (elements > 0 && (!d_values || !d_out)))
        return fail(RNS_ERR_INVALID_ARGUMENT, "encode: NULL pointer or negative size");
    if (elements == 0) return RNS_OK;
    encode_canonical_kernel<<<grid_for(elements, 256), 256, 0, as_stream(stream)>>>(
        d_values, d_out, modlist(pl), elements);
    RNS_CUDA_OK(cudaGetLastError());
    return RNS_OK;
}

int rns_encode_centered(const void* d_values, rns_int_type type, int64_t elements,
                        const int32_t* moduli, int channels, int8_t* d_out, rns_stream_t stream) {
    Plan pl;
    if (int rc = build_plan(moduli, channels, &pl)) return rc;
    if (elements < 0 || (elements > 0 && (!d_values || !d_out)))
        return fail(RNS_ERR_INVALID_ARGUMENT, "encode: NULL pointer or negative size");
    if (elements == 0) return RNS_OK;
    const int blocks = grid_for(elements, 256);
    cudaStream_t st = as_stream(stream);
    const ModList ml = modlist(pl);
    switch (type) {
        case RNS_INT8:
            encode_centered_kernel<int8_t><<<blocks, 256, 0, st>>>(
                static_cast<const int8_t*>(d_values), d_out, ml, elements);
            break;
        case RNS_INT16:
            encode_centered_kernel<int16_t><<<blocks, 256, 0, st>>>(
                static_cast<const int16_t*>(d_values), d_out, ml, elements);
            break;
        case RNS_INT32:
            encode_centered_kernel<int32_t><<<blocks, 256, 0, st>>>(
                static_cast<const int32_t*>(d_values), d_out, ml, elements);
            break;
        default:
            return fail(RNS_ERR_INVALID_ARGUMENT, "centered encoder supports int8, int16 and int32");
    }
    RNS_CUDA_OK(cudaGetLastError());
    return RNS_OK;
}

int rns_matmul_canonical_planes(const uint8_t* d_a, const uint8_t* d_b, const int32_t* moduli,
                                int channels, int m, int k, int n, int kernel_id, uint8_t* d_out,
                                rns_stream_t stream) {
    Plan pl;
    if (int rc = build_plan(moduli, channels, &pl)) return rc;
    if (int rc = check_gemm_dims(d_a, d_b, d_out, m, k, n)) return rc;
    if (kernel_id < 0 || kernel_id > 2)
        return fail(RNS_ERR_INVALID_ARGUMENT, "kernel_id must be 0, 1 or 2");
    return launch_plane_gemm<0>(d_a, d_b, d_out, pl, m, k, n, as_stream(stream));
}

int rns_matmul_centered_planes(const int8_t* d_a, const int8_t* d_b, const int32_t* moduli,
                               int channels, int m, int k, int n, int kernel_id, int8_t* d_out,
                               rns_stream_t stream) {
    Plan pl;
    if (int rc = build_plan(moduli, channels, &pl)) return rc;
    if (int rc = check_gemm_dims(d_a, d_b, d_out, m, k, n)) return rc;
    if (kernel_id < 0 || kernel_id > 3)
        return fail(RNS_ERR_INVALID_ARGUMENT,
                    "centered kernel_id must be scalar=0, dp4a=1, dp4a_safe=2 or cublas=3");
    if (kernel_id == 3 && (k % 4 != 0 || n % 4 != 0))
        return fail(RNS_ERR_INVALID_ARGUMENT,
                    "cuBLAS int8 path requires K and N to be multiples of 4");
    return launch_plane_gemm<1>(d_a, d_b, d_out, pl, m, k, n, as_stream(stream));
}

int rns_decode_garner(const int8_t* d_residues, int64_t elements, const int32_t* moduli,
                      int channels, int64_t* d_out, rns_stream_t stream) {
    Plan pl;
    if (int rc = build_plan(moduli, channels, &pl)) return rc;
    if (elements < 0 || (elements > 0 && (!d_residues || !d_out)))
        return fail(RNS_ERR_INVALID_ARGUMENT, "decode: NULL pointer or negative size");
    if (elements == 0) return RNS_OK;
    return launch_garner<int8_t>(d_residues, d_out, pl, elements, as_stream(stream));
}

int rns_matmul_centered_fused_out(const int8_t* d_a, const int8_t* d_b, const int32_t* moduli,
                                  int channels, int m, int k, int n, int lut_channels,
                                  int32_t* d_accumulators, int64_t* d_out, rns_stream_t stream) {
    Plan pl;
    if (int rc = build_plan(moduli, channels, &pl)) return rc;
    if (int rc = check_gemm_dims(d_a, d_b, d_out, m, k, n)) return rc;
    if (!d_accumulators) return fail(RNS_ERR_INVALID_ARGUMENT, "accumulator workspace is NULL");
    if (k % 4 != 0 || n % 4 != 0)
        return fail(RNS_ERR_INVALID_ARGUMENT, "fused path requires K and N multiples of 4");
    if (channels < 2 || channels > 10)
        return fail(RNS_ERR_UNSUPPORTED, "fused Garner path supports 2..10 channels");
    if (lut_channels < 0 || lut_channels > 2 || lut_channels > channels)
        return fail(RNS_ERR_INVALID_ARGUMENT,
                    "lut_channels must be 0, 1 or 2 and <= channel count");
    cudaStream_t st = as_stream(stream);
    if (int rc = launch_plane_gemm<2>(d_a, d_b, d_accumulators, pl, m, k, n, st)) return rc;
    return launch_garner<int32_t>(d_accumulators, d_out, pl, (int64_t)m * n, st);
}

static int quantize_impl(const void* d_x, rns_float_type type, int m, int k, int64_t ldx,
                         int col_block, int64_t col_block_stride,
                         int per_row, int quant_max, const int32_t* moduli, int channels,
                         int8_t* d_q, int8_t* d_planes, int packed_out, int tile_rows, float* d_scale,
                         int32_t* d_row_l1_max, void* d_scratch,
                         const uint32_t* d_absmax_parts, int absmax_parts, int64_t absmax_part_stride,
                         rns_stream_t stream) {
    if (!d_x || !d_scale || (!d_q && !d_planes))
        return fail(RNS_ERR_INVALID_ARGUMENT, "quantize: NULL pointer");
    if (col_block <= 0) { col_block = k; col_block_stride = 0; }
    if (m <= 0 || k <= 0 || ldx < col_block || k % col_block != 0)
        return fail(RNS_ERR_INVALID_ARGUMENT, "quantize: bad shape, stride or column block");
    // 127: int8 values (d_q) and / or their residue planes.  128..32767 (quant_bits 12 / 16 of the
    // reference's RNSLinear): residue planes only - the values themselves do not fit d_q.
    const bool wide = quant_max > 127;
    if (quant_max < 127 || quant_max > 32767 || (wide && (d_q != nullptr || d_planes == nullptr || d_row_l1_max != nullptr)))
        return fail(RNS_ERR_UNSUPPORTED, "the fused quantiser produces 8-bit values (quant_max 127), or residue planes "
                                         "only for quant_max up to 32767");
    if (tile_rows == 0) tile_rows = kPackM;
    if (tile_rows != kPackM && (!packed_out || d_q != nullptr || tile_rows < 8 || tile_rows > 128 || tile_rows % 8 != 0))
        return fail(RNS_ERR_INVALID_ARGUMENT, "quantize: tile_rows applies to packed planes only (multiple of 8, <= 128)");
    const bool given_absmax = d_absmax_parts != nullptr;
    if (given_absmax && (per_row || absmax_parts < 1 || absmax_parts > 64))
        return fail(RNS_ERR_INVALID_ARGUMENT, "quantize: a given absmax serves the per-tensor scale (1..64 parts)");
    // one CTA: beyond this size the two-launch path is faster
    const bool small = !per_row && !given_absmax && tile_rows == kPackM && (int64_t)m * k <= 32 * 1024;
    if (!per_row && !small && !given_absmax && !d_scratch)
        return fail(RNS_ERR_INVALID_ARGUMENT, "quantize: per-tensor scale needs d_scratch");
    if (packed_out && k % 8 != 0)
        return fail(RNS_ERR_INVALID_ARGUMENT, "quantize: the packed layout needs K % 8 == 0");
    QuantOut qo{};
    qo.q = d_q; qo.planes = d_planes; qo.scale = d_scale; qo.row_l1_max = d_row_l1_max;
    qo.packed = packed_out ? 1 : 0;
    qo.kblocks = (k + kPackK - 1) / kPackK;
    qo.tile_rows = tile_rows;
    if (d_planes)
        if (int rc = fill_encoder(qo, moduli, channels)) return rc;
#ifndef RNS_QUANT_CENTRED
    qo.reduced = (d_planes && packed_out) ? 1 : 0;   // the packed planes only feed the tensor cores
#endif
    if (wide) { qo.reduced = 0; qo.single_fold = 0; qo.fast = 0; }   // true centred residues of 16-bit integers
    size_t esize = 2;
    if (type == RNS_F32) esize = 4;
    else if (type != RNS_F16 && type != RNS_BF16)
        return fail(RNS_ERR_INVALID_ARGUMENT, "quantize: unknown float type");
    SrcView sv{};
    sv.x = d_x; sv.m = m; sv.k = k; sv.ldx = ldx;
    sv.col_block = col_block; sv.col_block_stride = col_block_stride;
    // every group of 8 columns contiguous and 16-byte aligned
    sv.vec8 = (k % 8 == 0 && col_block % 8 == 0 && (ldx * esize) % 16 == 0 &&
               (col_block_stride * esize) % 16 == 0 &&
               (reinterpret_cast<uintptr_t>(d_x) % 16) == 0) ? 1 : 0;
    cudaStream_t st = as_stream(stream);
    unsigned* scratch = static_cast<unsigned*>(d_scratch);
    const bool own_pass = !per_row && !small && !given_absmax;
    if (own_pass) RNS_CUDA_OK(cudaMemsetAsync(scratch, 0, 16, st));
    if (d_row_l1_max && !small) RNS_CUDA_OK(cudaMemsetAsync(d_row_l1_max, 0, sizeof(int32_t), st));
    const int row_threads = 128, seg_groups = 128, row_cap = 148 * 16;   // 1024-column segments
    int segments = 1;
    if (!per_row && !d_row_l1_max) segments = ((k + 7) / 8 + seg_groups - 1) / seg_groups;
    const int row_blocks = grid_for((int64_t)m * segments, row_threads / 32, row_cap);  // one warp per row segment
    const int64_t groups = (int64_t)m * ((k + 7) / 8);
    const unsigned* absmax_src = given_absmax ? d_absmax_parts : scratch;
    const int parts = given_absmax ? absmax_parts : 1;
    const int64_t part_stride = given_absmax ? absmax_part_stride : 0;
#define RNS_QUANT(T)                                                                           \
    do {                                                                                       \
        if (per_row) {                                                                         \
            quantize_rows_kernel<T, true><<<row_blocks, row_threads, 0, st>>>(sv, qo, quant_max, scratch, 1, 0, 1, 0); \
        } else if (small) {                                                                    \
            quantize_small_kernel<T><<<1, 1024, 0, st>>>(sv, qo, quant_max);                   \
        } else {                                                                               \
            if (own_pass) absmax_kernel<T><<<grid_for(groups, 256 * 4, 148 * 8), 256, 0, st>>>(sv, scratch); \
            quantize_rows_kernel<T, false><<<row_blocks, row_threads, 0, st>>>(sv, qo, quant_max, absmax_src, parts, part_stride, segments, seg_groups); \
        }                                                                                      \
    } while (0)
    switch (type) {
        case RNS_F16: RNS_QUANT(__half); break;
        case RNS_BF16: RNS_QUANT(__nv_bfloat16); break;
        default: RNS_QUANT(float); break;
    }
#undef RNS_QUANT
    RNS_CUDA_OK(cudaGetLastError());
    return RNS_OK;
}

int rns_quantize_activations(const void* d_x, rns_float_type type, int m, int k, int64_t ldx,
                             int col_block, int64_t col_block_stride,
                             int per_row, int quant_max, const int32_t* moduli, int channels,
                             int8_t* d_q, int8_t* d_planes, int packed_out, float* d_scale,
                             int32_t* d_row_l1_max, void* d_scratch, rns_stream_t stream) {
    return quantize_impl(d_x, type, m, k, ldx, col_block, col_block_stride, per_row, quant_max, moduli, channels,
                         d_q, d_planes, packed_out, 0, d_scale, d_row_l1_max, d_scratch, nullptr, 0, 0, stream);
}

int rns_quantize_activations_tiled(const void* d_x, rns_float_type type, int m, int k, int64_t ldx,
                                   int col_block, int64_t col_block_stride,
                                   int per_row, int quant_max, const int32_t* moduli, int channels,
                                   int8_t* d_q, int8_t* d_planes, int packed_out, int tile_rows, float* d_scale,
                                   int32_t* d_row_l1_max, void* d_scratch,
                                   const uint32_t* d_absmax_parts, int absmax_parts, int64_t absmax_part_stride,
                                   rns_stream_t stream) {
    return quantize_impl(d_x, type, m, k, ldx, col_block, col_block_stride, per_row, quant_max, moduli, channels,
                         d_q, d_planes, packed_out, tile_rows, d_scale, d_row_l1_max, d_scratch,
                         d_absmax_parts, absmax_parts, absmax_part_stride, stream);
}

int64_t rns_packed_weight_bytes(int n, int k) {
    if (n <= 0 || k <= 0) return 0;
    return round_up_i64(k, kPackK) * round_up_i64(n, kPackNPad);
}

int64_t rns_packed_planes_bytes(int m, int k, int channels, int tile_rows) {
    if (m <= 0 || k <= 0 || channels <= 0 || tile_rows <= 0) return 0;
    return round_up_i64(m, 2 * tile_rows) * round_up_i64(k, kPackK) * channels;
}

int64_t rns_packed_activation_bytes(int m, int k, int channels) {
    if (m <= 0 || k <= 0 || channels <= 0) return 0;
    // two row tiles at a time: a CTA pair always loads both, even past M
    return round_up_i64(m, 2 * kPackM) * round_up_i64(k, kPackK) * channels;
}

int rns_pack_weight(const int8_t* d_w, int n, int k, int64_t ldw, int8_t* d_packed, rns_stream_t stream) {
    if (!d_w || !d_packed) return fail(RNS_ERR_INVALID_ARGUMENT, "pack_weight: NULL pointer");
    if (n <= 0 || k <= 0 || ldw < k) return fail(RNS_ERR_INVALID_ARGUMENT, "pack_weight: bad shape or stride");
    const int64_t n_pad = round_up_i64(n, kPackNPad);
    const int kblocks = (k + kPackK - 1) / kPackK;
    pack_weight_kernel<false><<<grid_for(n_pad * kblocks * 4, 256), 256, 0, as_stream(stream)>>>(
        const_cast<int8_t*>(d_w), d_packed, n, k, ldw, n_pad, kblocks);
    RNS_CUDA_OK(cudaGetLastError());
    return RNS_OK;
}

int rns_unpack_weight(const int8_t* d_packed, int n, int k, int8_t* d_w, int64_t ldw, rns_stream_t stream) {
    if (!d_w || !d_packed) return fail(RNS_ERR_INVALID_ARGUMENT, "unpack_weight: NULL pointer");
    if (n <= 0 || k <= 0 || ldw < k) return fail(RNS_ERR_INVALID_ARGUMENT, "unpack_weight: bad shape or stride");
    const int64_t n_pad = round_up_i64(n, kPackNPad);
    const int kblocks = (k + kPackK - 1) / kPackK;
    pack_weight_kernel<true><<<grid_for(n_pad * kblocks * 4, 256), 256, 0, as_stream(stream)>>>(
        d_w, const_cast<int8_t*>(d_packed), n, k, ldw, n_pad, kblocks);
    RNS_CUDA_OK(cudaGetLastError());
    return RNS_OK;
}

int rns_encode_planes_packed(const int8_t* d_a, int m, int k, int64_t lda, const int32_t* moduli,
                             int channels, int8_t* d_planes_packed, rns_stream_t stream) {
    return rns_encode_planes_tiled(d_a, m, k, lda, moduli, channels, kPackM, d_planes_packed, stream);
}

int rns_encode_planes_tiled(const int8_t* d_a, int m, int k, int64_t lda, const int32_t* moduli,
                            int channels, int tile_rows, int8_t* d_planes_packed, rns_stream_t stream) {
    if (!d_a || !d_planes_packed) return fail(RNS_ERR_INVALID_ARGUMENT, "encode_planes: NULL pointer");
    if (m <= 0 || k <= 0 || lda < k)
        return fail(RNS_ERR_INVALID_ARGUMENT, "encode_planes: bad shape or stride");
    if (tile_rows < 8 || tile_rows > 128 || tile_rows % 8 != 0)
        return fail(RNS_ERR_INVALID_ARGUMENT, "encode_planes: tile_rows must be a multiple of 8, at most 128");
    QuantOut qo{};
    if (int rc = fill_encoder(qo, moduli, channels)) return rc;
    qo.planes = d_planes_packed;
    qo.packed = 1;
    qo.tile_rows = tile_rows;
    qo.kblocks = (k + kPackK - 1) / kPackK;
    encode_planes_packed_kernel<<<grid_for((int64_t)m * ((k + 15) / 16), 256), 256, 0, as_stream(stream)>>>(
        d_a, m, k, lda, qo);
    RNS_CUDA_OK(cudaGetLastError());
    return RNS_OK;
}

int rns_row_l1_max_i8(const int8_t* d_a, int m, int k, int64_t lda, int32_t* d_row_l1_max,
                      rns_stream_t stream) {
    if (!d_a || !d_row_l1_max) return fail(RNS_ERR_INVALID_ARGUMENT, "row_l1_max: NULL pointer");
    if (m <= 0 || k <= 0 || lda < k)
        return fail(RNS_ERR_INVALID_ARGUMENT, "row_l1_max: bad shape or stride");
    cudaStream_t st = as_stream(stream);
    RNS_CUDA_OK(cudaMemsetAsync(d_row_l1_max, 0, sizeof(int32_t), st));
    row_l1_max_kernel<<<m < 148 * 8 ? m : 148 * 8, 256, 0, st>>>(d_a, m, k, lda, d_row_l1_max);
    RNS_CUDA_OK(cudaGetLastError());
    return RNS_OK;
}

int rns_select_channels(const int32_t* d_row_l1_max, int32_t max_abs_weight, const int32_t* moduli,
                        int channels, int min_channels, int32_t* d_active_channels,
                        int64_t* d_meta, int64_t* d_histogram, int32_t* d_status,
                        rns_stream_t stream) {
    Plan pl;
    if (int rc = build_plan(moduli, channels, &pl)) return rc;
    if (!d_row_l1_max || !d_active_channels)
        return fail(RNS_ERR_INVALID_ARGUMENT, "select_channels: NULL pointer");
    if (min_channels < 2 || min_channels > channels)
        return fail(RNS_ERR_INVALID_ARGUMENT, "min_channels must be between 2 and len(moduli)");
    if (max_abs_weight < 0)
        return fail(RNS_ERR_INVALID_ARGUMENT, "bounds must be non-negative");
    SelectArgs sa;
    sa.channels = channels;
    sa.min_channels = min_channels;
    sa.max_abs_weight = max_abs_weight;
    for (int i = 0; i <= kMaxCh; ++i) sa.product[i] = pl.product[i];
    select_channels_kernel<<<1, 32, 0, as_stream(stream)>>>(
        d_row_l1_max, sa, d_active_channels, reinterpret_cast<long long*>(d_meta),
        reinterpret_cast<long long*>(d_histogram), d_status);
    RNS_CUDA_OK(cudaGetLastError());
    return RNS_OK;
}

int rns_quantize_weight(const void* d_w, rns_float_type type, int n, int k, int64_t ldw,
                        int quant_max, int8_t* d_wq, float* d_scale, int32_t* d_max_abs,
                        rns_stream_t stream) {
    if (!d_w || !d_wq || !d_scale) return fail(RNS_ERR_INVALID_ARGUMENT, "quantize_weight: NULL pointer");
    if (n <= 0 || k <= 0 || ldw < k)
        return fail(RNS_ERR_INVALID_ARGUMENT, "quantize_weight: bad shape or stride");
    if (quant_max < 1 || quant_max > 127)
        return fail(RNS_ERR_UNSUPPORTED, "weights are quantised to at most 8 bits");
    cudaStream_t st = as_stream(stream);
    if (d_max_abs) RNS_CUDA_OK(cudaMemsetAsync(d_max_abs, 0, sizeof(int32_t), st));
    const int grid = n < 148 * 8 ? n : 148 * 8;
    switch (type) {
        case RNS_F16:
            quantize_weight_kernel<__half><<<grid, 256, 0, st>>>(
                static_cast<const __half*>(d_w), n, k, ldw, quant_max, d_wq, d_scale, d_max_abs);
            break;
        case RNS_BF16:
            quantize_weight_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(
                static_cast<const __nv_bfloat16*>(d_w), n, k, ldw, quant_max, d_wq, d_scale, d_max_abs);
            break;
        case RNS_F32:
            quantize_weight_kernel<float><<<grid, 256, 0, st>>>(
                static_cast<const float*>(d_w), n, k, ldw, quant_max, d_wq, d_scale, d_max_abs);
            break;
        default:
            return fail(RNS_ERR_INVALID_ARGUMENT, "quantize_weight: unknown float type");
    }
    RNS_CUDA_OK(cudaGetLastError());
    return RNS_OK;
}

}  // extern "C"
