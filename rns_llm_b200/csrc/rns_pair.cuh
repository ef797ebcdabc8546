// Pieces shared by the two-CTA kernels (rns_gemm_pair_sm100.cu, which encodes canonical
// weight residues per channel, and rns_gemm_pair_raw_sm100.cu, which feeds every channel
// the int8 weight itself): kernel parameters, the barrier block, the packed-fp32
// reconstruction, the tile raster and the feature-major epilogue.
#pragma once

#include "rns_common.cuh"
#include "rns_ptx.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <atomic>
#include <type_traits>

namespace rns {

constexpr int kPairEncWarps = 16;
constexpr int kPairGroups = 2;                     // encoder groups; group g encodes the stages st = g (mod 2)
constexpr int kPairGroupWarps = kPairEncWarps / kPairGroups;
constexpr int kPairGroupThreads = kPairGroupWarps * 32;
constexpr int kPairPlaneWarp = 2 + kPairEncWarps;  // the warp that loads planes
constexpr int kPairThreads = (3 + kPairEncWarps) * 32;
constexpr int kDoneRing = 8;                       // ring of "stage done" barriers (>= both ring depths)
constexpr uint32_t kPairOpTile = 128 * kPackK;     // one channel's weight operand tile
constexpr size_t kPairStageBytes = 4 * 2 * 8 * 128 * 2;   // staging of the row-wide stores (output copies)
constexpr int kPairChunks = 128 * 4 / kPairGroupThreads;   // 16-byte chunks of a weight tile per encoder thread

struct PairParams {
    Plan plan;
    int32_t m, n, k;
    int32_t kblocks;
    const int8_t* planes;      // [M_pad / (TOK/2)][kblocks][R][TOK/2][64]
    const int8_t* w;           // packed weights [kblocks][w_npad][64]
    int64_t w_npad;
    int64_t w_channel_stride;  // 0: one matrix (the int8 weight) for every channel; else bytes between the
                               // packed residue planes of the weight, one per channel
    int32_t n_ftiles;          // tiles of 256 features (per problem of a grouped call)
    int32_t n_ttiles;          // tiles of TOK tokens (per problem)
    // Grouped calls (groups > 1; the raw-weight kernel's plain form): `groups` independent
    // problems of the same m x k x n.  The planes are those of the [groups * m, k] matrix (m a
    // multiple of the token tile), the weight is the packed [groups * n, k] matrix (problem g
    // owns rows g * w_group_rows ..), the outputs lie out_group_stride elements apart.
    int32_t groups;
    int32_t w_group_rows;
    int64_t out_group_stride;
    int32_t band;              // feature tiles per raster band
    void* out;
    int64_t ldo;
    int32_t out_type;
    const float* row_scale;
    int32_t row_scale_stride;
    const float* col_scale;
    const float* bias;
    uint32_t* absmax_out;      // NULL, or device words: [0] atomicMax of the bit pattern of max |y|,
                               // [1] count of CTAs that have contributed (both cleared by the launch)
    // Column-sharded layers: the tile is also stored, at the same offsets, into the output
    // buffers of the other ranks (peer memory, plain stores), and the finished absmax word
    // into theirs.  n_copies = 0: p.out only.
    int32_t n_copies;
    int32_t copies_mc;         // the copy addresses are multicast addresses: multimem.st instead of plain stores
    void* out_copies[RNS_MAX_PEERS];
    uint32_t* absmax_copies[RNS_MAX_PEERS];
    const int32_t* active;     // NULL, or device int: only the first *active channels are computed (adaptive prefix)
    int32_t* status;
    int32_t* wait_info;
};

struct __align__(8) PairCtl {
    uint64_t full_op[kDoneRing];     // leader: the encoder groups of BOTH CTAs have written the operand slot
    uint64_t full_pl[kDoneRing];     // this CTA's plane half has landed (leader: and the peer's)
    uint64_t done[kDoneRing];        // the MMAs of the stage are complete (arrives in both CTAs)
    uint64_t acc_full;               // the tile's MMAs are complete (arrives in both CTAs)
    uint64_t tmem_free;              // leader: both CTAs' accumulators are drained (and zeroed, where the kernel zeroes)
    uint64_t first_issued;           // leader, raw-weight kernel: the tile's first stage (which overwrites) is issued
    uint32_t tmem_base;
    int abort;
    uint32_t absmax;
};


// ---------------------------------------------------------------------------
// The epilogue's reconstruction for two outputs at a time with packed fp32
// instructions (fma / mul / add .f32x2: two IEEE single-precision results per
// instruction on sm_100).  Same operations, same rounding and same order per lane as
// garner_digits / reconstruct32 / reconstruct in rns_common.cuh (which the host tests
// evaluate); only the instruction count halves.
// ---------------------------------------------------------------------------
struct F2 { float x, y; };
__device__ __forceinline__ unsigned long long f2_bits(F2 v) {
    return ((unsigned long long)__float_as_uint(v.y) << 32) | (unsigned long long)__float_as_uint(v.x);
}
__device__ __forceinline__ F2 f2_from(unsigned long long b) {
    F2 v; v.x = __uint_as_float((unsigned)b); v.y = __uint_as_float((unsigned)(b >> 32)); return v;
}
__device__ __forceinline__ F2 f2_splat(float s) { F2 v; v.x = s; v.y = s; return v; }
__device__ __forceinline__ F2 fma2(F2 a, F2 b, F2 c) {
    unsigned long long d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(f2_bits(a)), "l"(f2_bits(b)), "l"(f2_bits(c)));
    return f2_from(d);
}
__device__ __forceinline__ F2 mul2(F2 a, F2 b) {
    unsigned long long d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(f2_bits(a)), "l"(f2_bits(b)));
    return f2_from(d);
}
__device__ __forceinline__ F2 add2(F2 a, F2 b) {
    unsigned long long d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(f2_bits(a)), "l"(f2_bits(b)));
    return f2_from(d);
}

// Centred mixed-radix digits of two outputs (all R channels active).  RES: a0 / a1 hold
// residues in [0, 2m) already (canonical_residue / nonneg_residue) instead of int32 channel sums.
// PREFIX: only the first `act` channels carry the value (adaptive prefix); the digits of the
// others are zero.  Without PREFIX `act` is ignored and all R channels are used.
template <int R, bool RES = false, bool PREFIX = false>
__device__ __forceinline__ void garner_digits_x2(const int (&a0)[R], const int (&a1)[R], const Plan& pl, F2 (&digit)[R],
                                                 int act = R) {
    const F2 magic = f2_splat(kMagic), neg_magic = f2_splat(-kMagic);
#pragma unroll
    for (int i = 0; i < R; ++i) {
        F2 r;
        r.x = bits_to_float((RES ? a0[i] : loose_residue(a0[i], pl.mod[i], pl.recip[i])) + kMagicBits);
        r.y = bits_to_float((RES ? a1[i] : loose_residue(a1[i], pl.mod[i], pl.recip[i])) + kMagicBits);
        r = add2(r, neg_magic);                                   // small_int_to_float
        F2 t = (i == 0) ? r : mul2(r, f2_splat(pl.gscale[i]));
#pragma unroll
        for (int j = 0; j < i; ++j) t = fma2(f2_splat(pl.gneg[i][j]), digit[j], t);
        // centre_mod: q = (t * rcp + magic) - magic;  digit = -q * m + t
        const F2 q = add2(fma2(t, f2_splat(pl.rcpf[i]), magic), neg_magic);
        digit[i] = fma2(q, f2_splat(-pl.modf[i]), t);
        if (PREFIX && i >= act) digit[i] = f2_splat(0.0f);
    }
}

// reconstruct32 for two outputs (R <= 4, all channels active).
template <int R, bool RES = false, bool PREFIX = false>
__device__ __forceinline__ void reconstruct32_x2(const int (&a0)[R], const int (&a1)[R], const Plan& pl, int& x0, int& x1,
                                                 int act = R) {
    static_assert(R <= 4, "32-bit reconstruction covers at most four channels");
    F2 digit[R];
    garner_digits_x2<R, RES, PREFIX>(a0, a1, pl, digit, act);
    const F2 magic = f2_splat(kMagic);
    unsigned u0 = 0, u1 = 0;
    if constexpr (R == 4) {
        const F2 lo = add2(fma2(f2_splat(pl.modf[0]), digit[1], digit[0]), magic);
        const F2 hi = add2(fma2(f2_splat(pl.modf[2]), digit[3], digit[2]), magic);
        u0 = (unsigned)(float_to_bits(lo.x) - kMagicBits) + pl.place32[2] * (unsigned)(float_to_bits(hi.x) - kMagicBits);
        u1 = (unsigned)(float_to_bits(lo.y) - kMagicBits) + pl.place32[2] * (unsigned)(float_to_bits(hi.y) - kMagicBits);
    } else {
#pragma unroll
        for (int i = 0; i < R; ++i) {
            const F2 d = add2(digit[i], magic);
            u0 += pl.place32[i] * (unsigned)(float_to_bits(d.x) - kMagicBits);
            u1 += pl.place32[i] * (unsigned)(float_to_bits(d.y) - kMagicBits);
        }
    }
    const unsigned prod = (unsigned)pl.product[PREFIX ? act : R];
    const int half = (int)(prod >> 1);
    const int low = (int)((unsigned)half - prod + 1u);
    int s0 = (int)u0, s1 = (int)u1;
    if (s0 > half) s0 = (int)(u0 - prod); else if (s0 < low) s0 = (int)(u0 + prod);
    if (s1 > half) s1 = (int)(u1 - prod); else if (s1 < low) s1 = (int)(u1 + prod);
    x0 = s0; x1 = s1;
}

// reconstruct for two outputs (any R up to 8, all channels active).
template <int R, bool RES = false, bool PREFIX = false>
__device__ __forceinline__ void reconstruct64_x2(const int (&a0)[R], const int (&a1)[R], const Plan& pl, long long& x0, long long& x1,
                                                 int act = R) {
    F2 digit[R];
    garner_digits_x2<R, RES, PREFIX>(a0, a1, pl, digit, act);
    const F2 magic = f2_splat(kMagic);
    int lo0 = 0, lo1 = 0;
    long long v0 = 0, v1 = 0;
#pragma unroll
    for (int i = 0; i < R; ++i) {
        const F2 d = add2(digit[i], magic);
        const int d0 = float_to_bits(d.x) - kMagicBits, d1 = float_to_bits(d.y) - kMagicBits;
        if (i < 4) { lo0 += (int)pl.place32[i] * d0; lo1 += (int)pl.place32[i] * d1; }
        else { v0 += pl.place64[i] * (long long)d0; v1 += pl.place64[i] * (long long)d1; }
    }
    v0 += lo0; v1 += lo1;
    const long long prod = pl.product[PREFIX ? act : R], half = prod >> 1;
    if (v0 > half) v0 -= prod; else if (v0 < half - prod + 1) v0 += prod;
    if (v1 > half) v1 -= prod; else if (v1 < half - prod + 1) v1 += prod;
    x0 = v0; x1 = v1;
}

// Output tile of a cluster: its position in the raster and the CTA's share of it.
struct PairTile {
    int n0;      // first feature of this CTA (inside its group)
    int tok0;    // first token of the pair's tile (inside its group)
    int tt;      // token tile index (inside its group)
    int grp;     // problem of a grouped call (0 otherwise)
};

template <int TOK>
__device__ __forceinline__ PairTile pair_tile(const PairParams& p, int tile, uint32_t rank) {
    // Raster: feature tiles in bands; inside a band the token tiles advance slowest, so
    // the clusters working at the same time share a band of the weight (it stays in L2)
    // and a few token tiles, and every plane byte is read from DRAM once per band.
    PairTile t;
    t.grp = 0;
    if (p.groups > 1) {              // grouped call: the problems one after the other, each with its own raster
        const int per_group = p.n_ftiles * p.n_ttiles;
        t.grp = tile / per_group;
        tile -= t.grp * per_group;
    }
    const int per_band = p.band * p.n_ttiles;
    const int band_i = tile / per_band;
    const int in_band = tile - band_i * per_band;
    const int band_w = min(p.band, p.n_ftiles - band_i * p.band);
    t.tt = in_band / band_w;
    const int ft = band_i * p.band + (in_band - t.tt * band_w);
    t.n0 = ft * 256 + (int)rank * 128;
    t.tok0 = t.tt * TOK;
    return t;
}

// Epilogue of one tile for one warp, feature-major: the warp owns tensor-memory lanes
// 32*quarter .. +31 (one output feature per lane) and the token columns
// part*TOK/4 .. +TOK/4 of every channel block.  Reads the R int32 sums of each output,
// reconstructs the integer, scales, converts and stores (also into the other ranks'
// buffers when COPIES); `biggest` collects max |y| of the stored values.
//
// SPLIT (up to four channels): two phases.  The first only empties tensor memory: every
// sum becomes its canonical residue, the R residues of an output share one register
// (a byte each), and `release()` runs as soon as the last column is read - the next
// tile's MMAs start then.  The second phase reconstructs, scales and stores from those
// registers while the tensor pipe is busy again.  Without SPLIT, release() runs last.
// PREFIX: `act` <= R channels carry the value (the adaptive prefix chosen on the device).
template <int R, int TOK, bool COPIES, bool SPLIT, bool PREFIX = false, typename Release>
__device__ __forceinline__ void pair_epilogue(const PairParams& p, int n0, int tok0, int quarter, int part, int lane,
                                              uint32_t lane_base, bool is_float, float rs_all, float& biggest,
                                              Release&& release, unsigned short* stage = nullptr, int act = R,
                                              int64_t out_off = 0) {
    static_assert(!SPLIT || R <= 6, "the packed form covers up to six channels");
    const int feat = n0 + quarter * 32 + lane;
    const bool feat_ok = feat < p.n;
    float cs = 0.0f, bs = 0.0f;
    if (is_float && feat_ok) {
        cs = p.col_scale[feat];
        if (p.bias != nullptr) bs = p.bias[feat];
    }
    using XInt = typename std::conditional<(R <= 4), int, long long>::type;
    constexpr int kColsPerPart = TOK / 4;
    // Two-byte outputs leave in pairs: lanes 2j and 2j+1 hold neighbouring features,
    // the even lane stores both features of the even tokens, the odd lane those of the
    // odd tokens (one 4-byte store instead of two 2-byte ones).
    bool pair_store = (p.out_type == RNS_OUT_F16 || p.out_type == RNS_OUT_BF16) && (p.ldo & 1) == 0 &&
                      (reinterpret_cast<uintptr_t>(p.out) & 3) == 0 && n0 + quarter * 32 + 32 <= p.n;
    for (int g = 0; COPIES && g < p.n_copies; ++g) pair_store = pair_store && (reinterpret_cast<uintptr_t>(p.out_copies[g]) & 3) == 0;
    // Row-wide stores (COPIES with a staging buffer): the four warps that share a block of
    // token columns (one per lane quarter, 4 x 32 features) meet in shared memory, 8 tokens at
    // a time, and each lane then stores 16 bytes, a warp two token rows of 256 contiguous
    // bytes - instead of 64-byte pieces, which NVLink carries at a fraction of its rate.
    bool wide_store = false;
    if constexpr (COPIES) {
        wide_store = stage != nullptr && (p.out_type == RNS_OUT_F16 || p.out_type == RNS_OUT_BF16) &&
                     n0 + 128 <= p.n && (p.ldo & 7) == 0 && (reinterpret_cast<uintptr_t>(p.out) & 15) == 0;
        for (int g = 0; g < p.n_copies; ++g)
            wide_store = wide_store && (reinterpret_cast<uintptr_t>(p.out_copies[g]) & 15) == 0;
    }
    auto load = [&](int col, int (&acc)[R][8]) {
        __syncwarp();
#pragma unroll
        for (int c = 0; c < R; ++c) tmem_ld8(lane_base + (uint32_t)(c * TOK + col), acc[c]);
    };
    auto finish = [&](int col, const int (&acc)[R][8], auto from_residues) {
        [[maybe_unused]] constexpr bool RES = decltype(from_residues)::value;
        const int tok_first = tok0 + col;
        if (tok_first >= p.m) return;                  // warp-uniform
        XInt xv[8];
#pragma unroll
        for (int t8 = 0; t8 < 8; t8 += 2) {
            int one0[R], one1[R];
#pragma unroll
            for (int c = 0; c < R; ++c) { one0[c] = acc[c][t8]; one1[c] = acc[c][t8 + 1]; }
            if constexpr (R <= 4) reconstruct32_x2<R, RES, PREFIX>(one0, one1, p.plan, xv[t8], xv[t8 + 1], act);
            else reconstruct64_x2<R, RES, PREFIX>(one0, one1, p.plan, xv[t8], xv[t8 + 1], act);
        }
        const int valid_t = min(8, p.m - tok_first);   // warp-uniform
        if (!is_float) {
            if (!feat_ok) return;
#pragma unroll
            for (int t8 = 0; t8 < 8; ++t8) {
                if (t8 < valid_t) {
                    const int64_t o = out_off + (int64_t)(tok_first + t8) * p.ldo + feat;
                    if (p.out_type == RNS_OUT_INT64) static_cast<long long*>(p.out)[o] = (long long)xv[t8];
                    else static_cast<int*>(p.out)[o] = (int)xv[t8];
                }
            }
            return;
        }
        float y[8];
#pragma unroll
        for (int t8 = 0; t8 < 8; t8 += 2) {
            F2 xf, rs;
            if constexpr (R <= 4) { xf.x = __int2float_rn(xv[t8]); xf.y = __int2float_rn(xv[t8 + 1]); }
            else { xf.x = __ll2float_rn(xv[t8]); xf.y = __ll2float_rn(xv[t8 + 1]); }
            rs.x = p.row_scale_stride == 0 ? rs_all : (t8 < valid_t ? p.row_scale[tok_first + t8] : 0.0f);
            rs.y = p.row_scale_stride == 0 ? rs_all : (t8 + 1 < valid_t ? p.row_scale[tok_first + t8 + 1] : 0.0f);
            F2 v = mul2(mul2(xf, rs), f2_splat(cs));       // separately rounded, in the reference's order
            if (p.bias != nullptr) v = add2(v, f2_splat(bs));
            y[t8] = v.x; y[t8 + 1] = v.y;
        }
        if (p.out_type == RNS_OUT_F32) {
            if (!feat_ok) return;
#pragma unroll
            for (int t8 = 0; t8 < 8; ++t8) {
                if (t8 < valid_t) {
                    const int64_t o = out_off + (int64_t)(tok_first + t8) * p.ldo + feat;
                    static_cast<float*>(p.out)[o] = y[t8];
                    for (int g = 0; COPIES && g < p.n_copies; ++g) static_cast<float*>(p.out_copies[g])[o] = y[t8];
                    biggest = fmaxf(biggest, fabsf(y[t8]));
                }
            }
            return;
        }
        // fp16 / bf16: the stored bit patterns, and their magnitudes for the absmax word
        unsigned short h[8];
#pragma unroll
        for (int t8 = 0; t8 < 8; ++t8) {
            if (p.out_type == RNS_OUT_F16) {
                const __half v = __float2half_rn(y[t8]);
                h[t8] = __half_as_ushort(v);
                if (t8 < valid_t && feat_ok) biggest = fmaxf(biggest, fabsf(__half2float(v)));
            } else {
                const __nv_bfloat16 v = __float2bfloat16_rn(y[t8]);
                h[t8] = __bfloat16_as_ushort(v);
                if (t8 < valid_t && feat_ok) biggest = fmaxf(biggest, fabsf(__bfloat162float(v)));
            }
        }
        unsigned short* out16 = static_cast<unsigned short*>(p.out);
        if (COPIES && wide_store) {
            // two buffers per token-column block: a buffer is rewritten two chunks later, after
            // every one of the four warps has passed the barrier of the chunk in between
            const int chunk = (col - part * kColsPerPart) >> 3;
            unsigned short* sb = stage + ((part * 2 + (chunk & 1)) * 8) * 128;
#pragma unroll
            for (int t8 = 0; t8 < 8; ++t8) sb[t8 * 128 + quarter * 32 + lane] = h[t8];
            asm volatile("bar.sync %0, 128;" ::"r"(2 + part) : "memory");
            const int t = quarter * 2 + (lane >> 4);
            const uint4 v = *reinterpret_cast<const uint4*>(sb + t * 128 + (lane & 15) * 8);
            if (t < valid_t) {
                const int64_t o = out_off + (int64_t)(tok_first + t) * p.ldo + n0 + (lane & 15) * 8;
                *reinterpret_cast<uint4*>(out16 + o) = v;
                for (int g = 0; g < p.n_copies; ++g) {
                    unsigned short* dst = static_cast<unsigned short*>(p.out_copies[g]) + o;
                    if (p.copies_mc) multimem_store16(dst, v);      // one store, every rank of the multicast group
                    else *reinterpret_cast<uint4*>(dst) = v;
                }
            }
            return;
        }
        if (pair_store) {
            const bool odd = (lane & 1) != 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                // even lane keeps token 2i and sends token 2i+1; odd lane the other way round
                const unsigned mine = odd ? h[2 * i + 1] : h[2 * i];
                const unsigned send = odd ? h[2 * i] : h[2 * i + 1];
                const unsigned got = __shfl_xor_sync(0xffffffffu, send, 1);
                const int t8 = 2 * i + (odd ? 1 : 0);
                if (t8 < valid_t) {
                    const unsigned word = odd ? (got | (mine << 16)) : (mine | (got << 16));
                    const int64_t o = out_off + (int64_t)(tok_first + t8) * p.ldo + (feat & ~1);
                    *reinterpret_cast<unsigned*>(out16 + o) = word;
                    for (int g = 0; COPIES && g < p.n_copies; ++g)
                        *reinterpret_cast<unsigned*>(static_cast<unsigned short*>(p.out_copies[g]) + o) = word;
                }
            }
        } else if (feat_ok) {
#pragma unroll
            for (int t8 = 0; t8 < 8; ++t8) {
                if (t8 < valid_t) {
                    const int64_t o = out_off + (int64_t)(tok_first + t8) * p.ldo + feat;
                    out16[o] = h[t8];
                    for (int g = 0; COPIES && g < p.n_copies; ++g) static_cast<unsigned short*>(p.out_copies[g])[o] = h[t8];
                }
            }
        }
    };
    const int col0 = part * kColsPerPart;
    constexpr int kIters = kColsPerPart / 8;
    const std::false_type sums;
    if constexpr (SPLIT) {
        // Phase 1.  One buffer: the other warps of the scheduler cover the load latency.
        // Channels 0..3 of an output share one register, a byte each; channels 4 and 5 are
        // packed densely, kExtra bytes per output, 8 * kExtra bytes per step of 8 columns.
        constexpr int kLow = R < 4 ? R : 4;
        constexpr int kExtra = R - kLow;
        constexpr int kHighWords = kExtra == 0 ? 1 : 2 * kExtra;
        uint32_t packed[kIters][8];
        [[maybe_unused]] uint32_t packed_high[kIters][kHighWords];
        // Every modulus below 128 (the int8 configurations): the Barrett step's result in
        // [0, 2m) already fits its byte, and the recurrence of phase 2 takes it as it is.
        const bool byte_fits = p.plan.encode_fast != 0;
        auto residue = [&](int v, int c) -> uint32_t {
            return byte_fits ? nonneg_residue(v, p.plan.mod[c], p.plan.recip[c], p.plan.ubias[c])
                             : canonical_residue(v, p.plan.mod[c], p.plan.recip[c], p.plan.ubias[c]);
        };
#pragma unroll
        for (int it = 0; it < kIters; ++it) {
            int acc[R][8];
            load(col0 + it * 8, acc);
            tmem_ld_wait();
#pragma unroll
            for (int w = 0; w < kHighWords; ++w) packed_high[it][w] = 0u;
#pragma unroll
            for (int t8 = 0; t8 < 8; ++t8) {
                uint32_t word = 0;
#pragma unroll
                for (int c = 0; c < kLow; ++c)
                    if (!PREFIX || c < act)      // columns of unused channels hold stale sums
                        word |= residue(acc[c][t8], c) << (8 * c);
                packed[it][t8] = word;
#pragma unroll
                for (int e = 0; e < kExtra; ++e) {
                    const int byte = t8 * kExtra + e;                // position in this step's high bytes
                    if (!PREFIX || kLow + e < act)
                        packed_high[it][byte >> 2] |= residue(acc[kLow + e][t8], kLow + e) << (8 * (byte & 3));
                }
            }
        }
        release();
        // Phase 2.
        const std::true_type residues;
#pragma unroll
        for (int it = 0; it < kIters; ++it) {
            int acc[R][8];
#pragma unroll
            for (int t8 = 0; t8 < 8; ++t8) {
#pragma unroll
                for (int c = 0; c < kLow; ++c) acc[c][t8] = (int)((packed[it][t8] >> (8 * c)) & 0xffu);
#pragma unroll
                for (int e = 0; e < kExtra; ++e) {
                    const int byte = t8 * kExtra + e;
                    acc[kLow + e][t8] = (int)((packed_high[it][byte >> 2] >> (8 * (byte & 3))) & 0xffu);
                }
            }
            finish(col0 + it * 8, acc, residues);
        }
    } else if constexpr (R <= 4) {
        // The loads of the next 8 token columns are in flight while these are finished.
        int a0[R][8], a1[R][8];
        load(col0, a0);
#pragma unroll
        for (int it = 0; it < kIters; it += 2) {
            tmem_ld_wait();
            if (it + 1 < kIters) load(col0 + (it + 1) * 8, a1);
            finish(col0 + it * 8, a0, sums);
            if (it + 1 < kIters) {
                tmem_ld_wait();
                if (it + 2 < kIters) load(col0 + (it + 2) * 8, a0);
                finish(col0 + (it + 1) * 8, a1, sums);
            }
        }
        release();
    } else {
        // one buffer: two of them (2 x R x 8 registers) would spill
#pragma unroll 1
        for (int it = 0; it < kIters; ++it) {
            int acc[R][8];
            load(col0 + it * 8, acc);
            tmem_ld_wait();
            finish(col0 + it * 8, acc, sums);
        }
        release();
    }
}

// Launches a persistent two-CTA-cluster kernel: as many clusters as the device holds at
// once (one CTA per SM; a GPC with an odd number of SMs leaves one unpaired), at most one
// per tile.  The opt-in shared-memory size and the resident count are found once per
// device and kernel.
template <void (*Kernel)(PairParams)>
static int launch_pair_clusters(size_t smem, const PairParams& pp, int pairs, cudaStream_t st) {
    static std::atomic<int> resident[64];
    int dev = 0;
    RNS_CUDA_OK(cudaGetDevice(&dev));
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.blockDim = dim3(kPairThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int clusters = resident[dev & 63].load(std::memory_order_acquire);
    if (clusters == 0) {
        RNS_CUDA_OK(cudaFuncSetAttribute(Kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        int sms = 0;
        RNS_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        cfg.gridDim = dim3((unsigned)(sms & ~1), 1, 1);
        if (cudaOccupancyMaxActiveClusters(&clusters, Kernel, &cfg) != cudaSuccess || clusters < 1) {
            cudaGetLastError();
            clusters = sms / 2 > 8 ? sms / 2 - 4 : 1;          // a safe guess: a few SMs short of all
        }
        resident[dev & 63].store(clusters, std::memory_order_release);
    }
    if (clusters > pairs) clusters = pairs;
    cfg.gridDim = dim3((unsigned)(2 * clusters), 1, 1);
    const cudaError_t rc = cudaLaunchKernelEx(&cfg, Kernel, pp);
    if (rc != cudaSuccess) {
        cudaGetLastError();
        return fail(RNS_ERR_CUDA, "launch of the paired RNS GEMM failed: %s (%d clusters for %d tiles, smem %zu)",
                    cudaGetErrorString(rc), clusters, pairs, smem);
    }
    return RNS_OK;
}

// rns_gemm_pair_raw_sm100.cu
int pair_raw_token_tile(int channels);
int launch_pair_raw_gemm(const PairParams& pp, int pairs, cudaStream_t st);

}  // namespace rns
