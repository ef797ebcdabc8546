// Fused RNS linear for sm_100a, large-M variant: the encoded weights never touch
// shared memory.
//
// rns_gemm_kernel (rns_gemm_sm100.cu) stages R encoded copies of every operand
// tile in shared memory, and its tensor-core operand reads, TMA writes and encoder
// traffic all go through the same 128 B/clk of shared-memory bandwidth; that, not
// the tensor pipe, bounds it.  Here the roles of the operands are swapped:
//
//   D^T[n, t] += W_c[n, :] . A_c[t, :]        per residue channel c
//
// * The weight tile (128 output features n) is the MMA's A operand and lives in
//   TENSOR MEMORY.  Worker warps read their rows' source bytes straight from
//   global memory (the packed weight layout makes that a coalesced 64 bytes per
//   thread and K block), form the R residues in registers and store them with
//   tcgen05.st: no TMA, no shared memory, no operand re-read.
// * The activation planes (the caller encodes them once per call) are the B
//   operand: one bulk copy per K block and channel set brings TT tokens x 64 bytes
//   x R planes into a shared-memory ring, which is all the shared-memory traffic
//   that is left (written once, read once by the MMAs).
// * R accumulators of 128 x TT int32 sit in tensor memory next to a ring of four
//   weight-operand slots (16 columns per slot and channel).
// * The epilogue is the same arithmetic on transposed tiles: a thread owns one
//   output feature and walks the tokens; a warp stores 32 consecutive features of
//   one token at a time.
//
// Warp roles (576 threads): warp 0 plane producer (one lane), warp 1 tensor-memory
// owner and MMA issuer (one lane), warps 2..17 workers.  Worker warp w serves lane
// quarter w & 3 (32 weight rows) and K blocks kb = (w - 2) / 4 (mod 4): four groups
// of four warps, each group with its own operand slot, so a slot's hand-over
// latency overlaps with the other groups' encoding.  Hand-overs to the MMA lane
// happen per PAIR of K blocks.
//
// Every mbarrier wait is bounded, as in rns_gemm_kernel.
#include "rns_common.cuh"
#include "rns_ptx.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <atomic>
#include <type_traits>

namespace rns {

constexpr int kV2Threads = 576;
constexpr int kV2Workers = 16;
constexpr int kV2Slots = 4;            // weight-operand slots (K blocks) in tensor memory
constexpr int kV2SlotPairs = 2;        // hand-over granularity: two K blocks
constexpr int kV2MaxPlaneStages = 8;

struct TmemGemmParams {
    Plan plan;
    int32_t m, n, k;                   // tokens, output features, depth
    int32_t tile_t;                    // tokens per tile (MMA N): 128, 64 or 32
    int32_t plane_stages;              // shared-memory ring depth, in K-block pairs
    int32_t tmem_cols;                 // allocation (power of two)
    int32_t opnd_col0;                 // first column of the operand slots
    int32_t exact_residues;
    const int32_t* active_ptr;
    const int8_t* planes;              // packed [M_pad/128][K/64][R][128][64]
    const int8_t* w;                   // packed [K/64][N_pad][64]
    int64_t w_npad;
    void* out;
    int64_t ldo;
    int32_t out_type;
    const float* row_scale;
    int32_t row_scale_stride;
    const float* col_scale;
    const float* bias;
    int32_t* status;
    uint32_t plane_sub_bytes;          // one K block: R * tile_t * 64
};

struct __align__(8) V2Ctl {
    uint64_t pl_full[kV2MaxPlaneStages];    // planes of a K-block pair have landed
    uint64_t pl_empty[kV2MaxPlaneStages];   // ... and the MMAs that read them are done
    uint64_t op_full[kV2SlotPairs];         // weight operands of a K-block pair are in tensor memory
    uint64_t op_empty[kV2SlotPairs];        // ... and consumed
    uint64_t acc_full;
    uint32_t tmem_base;
    int abort;
};

// Encodes the 64 source bytes of one weight row (16 words) for channel c into v[].
template <int R>
__device__ __forceinline__ void encode_row_channel(const uint32_t (&x)[16], const uint32_t (&d)[16],
                                                   uint32_t mfold, uint32_t hi, uint32_t lo, uint32_t mk,
                                                   bool reduced, bool fast, uint32_t (&v)[16]) {
    if (reduced) {
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = encode_word_reduced(x[i] ^ 0x80808080u, d[i], mfold);
    } else if (fast) {
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = encode_word<true>(x[i] ^ 0x80808080u, x[i] & 0x7f7f7f7fu, hi, lo, mk);
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = encode_word<false>(x[i] ^ 0x80808080u, x[i] & 0x7f7f7f7fu, hi, lo, mk);
    }
}

template <int R>
__global__ void __launch_bounds__(kV2Threads, 1)
rns_gemm_tmem_kernel(const __grid_constant__ TmemGemmParams p) {
    extern __shared__ uint8_t smem_dyn[];
    __shared__ V2Ctl ctl;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t ring_base = (smem_addr(smem_dyn) + 1023u) & ~1023u;

    // grid: x = token tile (fastest: resident CTAs share one weight tile), y = feature tile
    const int t0 = blockIdx.x * p.tile_t;
    const int n0 = blockIdx.y * 128;
    const int kblocks = (p.k + 63) / 64;
    const int npairs = (kblocks + 1) / 2;
    const int TT = p.tile_t;
    const int stages = p.plane_stages;
    const uint32_t stage_bytes = 2u * p.plane_sub_bytes;

    int active = R;
    if (p.active_ptr != nullptr) {
        active = *p.active_ptr;
        active = active < 1 ? 1 : (active > R ? R : active);
    }

    if (threadIdx.x == 0) {
        ctl.abort = 0;
        for (int s = 0; s < kV2MaxPlaneStages; ++s) {
            mbar_init(smem_addr(&ctl.pl_full[s]), 1);
            mbar_init(smem_addr(&ctl.pl_empty[s]), 1);
        }
        for (int s = 0; s < kV2SlotPairs; ++s) {
            mbar_init(smem_addr(&ctl.op_full[s]), 8);    // two groups of four warps
            mbar_init(smem_addr(&ctl.op_empty[s]), 1);
        }
        mbar_init(smem_addr(&ctl.acc_full), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(smem_addr(&ctl.tmem_base), (uint32_t)p.tmem_cols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = ctl.tmem_base;
    volatile int* abort = &ctl.abort;

    if (warp == 0) {
        // ------------------------------ plane producer ----------------------------
        if (lane == 0) {
            // token tile inside the packed 128-row tile: rows [t0 % 128, +TT) of each plane
            const int64_t row_tile = t0 >> 7;
            const uint32_t row_off = (uint32_t)(t0 & 127) * kPackK;
            const uint32_t plane_bytes = (uint32_t)TT * kPackK;
            for (int pr = 0; pr < npairs; ++pr) {
                const int s = pr % stages;
                const uint32_t round = (uint32_t)(pr / stages);
                const uint32_t stage = ring_base + (uint32_t)s * stage_bytes;
                const int jn = min(2, kblocks - 2 * pr);
                if (round > 0 && !wait_bounded<false, true>(smem_addr(&ctl.pl_empty[s]), (round - 1) & 1, abort)) break;
                const uint32_t bar = smem_addr(&ctl.pl_full[s]);
                mbar_arrive_expect_tx(bar, (uint32_t)(jn * active) * plane_bytes);
                for (int j = 0; j < jn; ++j) {
                    const int kb = 2 * pr + j;
                    const int8_t* src = p.planes + ((row_tile * kblocks + kb) * R) * (int64_t)(kPackM * kPackK) + row_off;
                    for (int c = 0; c < active; ++c)
                        bulk_load(stage + (uint32_t)j * p.plane_sub_bytes + (uint32_t)c * plane_bytes,
                                  src + (int64_t)c * (kPackM * kPackK), plane_bytes, bar);
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------ MMA issuer --------------------------------
        if (lane == 0) {
            const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | (((uint32_t)TT >> 3) << 17) | (8u << 24);
            const uint32_t plane_bytes = (uint32_t)TT * kPackK;
            bool ok = true;
            for (int pr = 0; pr < npairs && ok; ++pr) {
                const int sp = pr % stages;
                const int so = pr % kV2SlotPairs;
                const uint32_t stage = ring_base + (uint32_t)sp * stage_bytes;
                const int jn = min(2, kblocks - 2 * pr);
                ok = wait_bounded<false, true>(smem_addr(&ctl.op_full[so]), (uint32_t)(pr / kV2SlotPairs) & 1, abort);
                if (ok) ok = wait_bounded<false, true>(smem_addr(&ctl.pl_full[sp]), (uint32_t)(pr / stages) & 1, abort);
                if (!ok) break;
                tc_fence_after();
                for (int j = 0; j < jn; ++j) {
                    const int slot = 2 * so + j;
                    for (int c = 0; c < active; ++c) {
                        const uint32_t d = tmem_base + (uint32_t)(c * TT);
                        const uint32_t a_col = tmem_base + (uint32_t)(p.opnd_col0 + (slot * R + c) * 16);
                        const uint32_t b_tile = stage + (uint32_t)j * p.plane_sub_bytes + (uint32_t)c * plane_bytes;
#pragma unroll
                        for (int ks = 0; ks < 2; ++ks)
                            umma_i8_ts(d, a_col + (uint32_t)(ks * 8), make_smem_desc(b_tile + ks * 32, 64), idesc,
                                       (pr > 0 || j > 0 || ks > 0) ? 1u : 0u);
                    }
                }
                umma_commit(smem_addr(&ctl.op_empty[so]));
                umma_commit(smem_addr(&ctl.pl_empty[sp]));
            }
            if (ok) umma_commit(smem_addr(&ctl.acc_full));
        }
        __syncwarp();
    } else {
        // ------------------------------ weight encoders ---------------------------
        const int quarter = warp & 3;                 // tensor-memory lanes 32*quarter .. +31
        const int group = (warp - 2) >> 2;            // K blocks kb = group (mod 4)
        const int row = n0 + quarter * 32 + lane;     // weight row of this thread (always inside N_pad)
        const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
        const bool reduced = p.exact_residues == 0;
        const bool fast = p.plan.encode_fast != 0;
        // chunk j of the row's 64 bytes is stored at chunk j ^ ((row >> 1) & 3)
        const int swz = (row >> 1) & 3;
        const int8_t* wrow = p.w + (int64_t)row * kPackK;
        const int64_t kb_stride = p.w_npad * kPackK;

        // Two K blocks of this thread's weight bytes are kept in registers ahead of use.
        uint4 cur[4], nxt[4];
        auto load_block = [&](int kb, uint4 (&dst)[4]) {
            const uint4* src = reinterpret_cast<const uint4*>(wrow + (int64_t)kb * kb_stride);
#pragma unroll
            for (int j = 0; j < 4; ++j) dst[j] = __ldg(src + (j ^ swz));
        };
        if (group < kblocks) load_block(group, cur);
        if (group + 4 < kblocks) load_block(group + 4, nxt);

        bool ok = true;
        for (int kb = group; kb < kblocks && ok; kb += 4) {
            const int pr = kb >> 1;
            const int so = pr % kV2SlotPairs;             // = group >> 1
            const int slot = 2 * so + (kb & 1);           // = group
            const uint32_t round = (uint32_t)(pr / kV2SlotPairs);
            uint32_t x[16];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                x[4 * j] = cur[j].x; x[4 * j + 1] = cur[j].y; x[4 * j + 2] = cur[j].z; x[4 * j + 3] = cur[j].w;
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) cur[j] = nxt[j];
            if (kb + 8 < kblocks) load_block(kb + 8, nxt);
            uint32_t d[16];
            if (reduced) {
#pragma unroll
                for (int i = 0; i < 16; ++i) d[i] = fold_pattern(x[i]);
            }
            // the slot pair must have been consumed by the MMAs of its previous revolution of the ring
            if (round > 0) ok = wait_bounded(smem_addr(&ctl.op_empty[so]), (round - 1) & 1, abort);
            if (!ok) break;
            tc_fence_after();
#pragma unroll
            for (int c = 0; c < R; ++c) {
                if (c < active) {
                    uint32_t v[16];
                    encode_row_channel<R>(x, d, p.plan.enc_mfold[c], p.plan.enc_hi[c], p.plan.enc_lo[c],
                                          p.plan.enc_mk[c], reduced, fast, v);
                    tmem_st16(lane_base + (uint32_t)(p.opnd_col0 + (slot * R + c) * 16), v);
                }
            }
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_addr(&ctl.op_full[so]));
        }
        // A K-block count that is not a multiple of four leaves some groups one
        // hand-over short of their partners in the last pair: every pair needs all
        // eight arrivals, so groups without a K block in the final pair arrive empty.
        // (pairs are complete except possibly the last one, which has one K block)
        if (ok && (kblocks & 1)) {
            const int last = kblocks - 1;                  // the lone K block of the last pair
            const int partner_group = (last + 1) & 3;      // group that would own its missing partner
            if (group == partner_group) {
                const int pr = last >> 1;
                const int so = pr % kV2SlotPairs;
                const uint32_t round = (uint32_t)(pr / kV2SlotPairs);
                if (round > 0) ok = wait_bounded(smem_addr(&ctl.op_empty[so]), (round - 1) & 1, abort);
                __syncwarp();
                if (ok && lane == 0) mbar_arrive(smem_addr(&ctl.op_full[so]));
            }
        }

        // ------------------------------ epilogue ----------------------------------
        if (ok) ok = wait_bounded(smem_addr(&ctl.acc_full), 0, abort);
        if (ok) {
            tc_fence_after();
            const int part = (warp - 2) >> 2;              // token chunks are dealt round-robin
            const bool is_float = p.out_type >= RNS_OUT_F16;
            const bool row_ok = row < p.n;
            float cs = 0.0f, bs = 0.0f;
            if (is_float && row_ok) {
                cs = p.col_scale[row];
                if (p.bias != nullptr) bs = p.bias[row];
            }
            using XInt = typename std::conditional<(R <= 4), int, long long>::type;
            for (int col = part * 8; col < TT; col += 32) {
                __syncwarp();
                int acc[R][8];
#pragma unroll
                for (int c = 0; c < R; ++c) {
                    if (c < active) {
                        tmem_ld8(lane_base + (uint32_t)(c * TT + col), acc[c]);
                    } else {
#pragma unroll
                        for (int e = 0; e < 8; ++e) acc[c][e] = 0;
                    }
                }
                tmem_ld_wait();
                const int tok0 = t0 + col;
                if (!row_ok || tok0 >= p.m) continue;
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const int tok = tok0 + e;
                    if (tok >= p.m) break;
                    int one[R];
#pragma unroll
                    for (int c = 0; c < R; ++c) one[c] = acc[c][e];
                    XInt xv;
                    if constexpr (R <= 4) xv = reconstruct32<R>(one, p.plan, active);
                    else xv = reconstruct<R>(one, p.plan, active);
                    const int64_t o = (int64_t)tok * p.ldo + row;
                    if (p.out_type == RNS_OUT_INT64) {
                        static_cast<long long*>(p.out)[o] = (long long)xv;
                    } else if (p.out_type == RNS_OUT_INT32) {
                        static_cast<int*>(p.out)[o] = (int)xv;
                    } else {
                        float xf;
                        if constexpr (R <= 4) xf = __int2float_rn(xv);
                        else xf = __ll2float_rn(xv);
                        const float rs = p.row_scale[(int64_t)tok * p.row_scale_stride];
                        float y = __fmul_rn(__fmul_rn(xf, rs), cs);
                        if (p.bias != nullptr) y = __fadd_rn(y, bs);
                        if (p.out_type == RNS_OUT_F16) static_cast<__half*>(p.out)[o] = __float2half_rn(y);
                        else if (p.out_type == RNS_OUT_BF16) static_cast<__nv_bfloat16*>(p.out)[o] = __float2bfloat16_rn(y);
                        else static_cast<float*>(p.out)[o] = y;
                    }
                }
            }
        }
    }

    // ------------------------------ teardown ---------------------------------------
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && ctl.abort && p.status != nullptr)
        atomicExch(p.status, (int)RNS_ERR_DEVICE_TIMEOUT);
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
    }
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
template <int R>
static int launch_tmem(const TmemGemmParams& gp, dim3 grid, size_t smem, cudaStream_t st) {
    static std::atomic<uint64_t> configured{0};
    int dev = 0;
    RNS_CUDA_OK(cudaGetDevice(&dev));
    const uint64_t bit = 1ull << (dev & 63);
    if (!(configured.load(std::memory_order_acquire) & bit)) {
        RNS_CUDA_OK(cudaFuncSetAttribute(rns_gemm_tmem_kernel<R>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         227 * 1024 - 1024));
        configured.fetch_or(bit, std::memory_order_release);
    }
    rns_gemm_tmem_kernel<R><<<grid, kV2Threads, smem, st>>>(gp);
    RNS_CUDA_OK(cudaGetLastError());
    return RNS_OK;
}

// 1 when the tensor-memory-operand kernel can run this problem: packed planes and
// packed weights, 2..5 channels.
bool tmem_gemm_supported(const rns_linear_args* a) {
    return a->d_a_planes != nullptr && a->a_packed && a->w_packed && a->channels >= 2 && a->channels <= 5 &&
           a->tile_k != 128;
}

int launch_tmem_gemm(const rns_linear_args* a, const Plan& plan, cudaStream_t st) {
    TmemGemmParams gp;
    memset(&gp, 0, sizeof(gp));
    gp.plan = plan;
    const int R = plan.channels;
    gp.m = a->m; gp.n = a->n; gp.k = a->k;
    // tokens per tile: accumulators take R*tile_t columns and must leave room for
    // four operand slots of R*16 columns each
    int tile_t = R <= 2 ? 128 : (R <= 4 ? 64 : 32);
    if (a->tile_n == 32 || a->tile_n == 64 || a->tile_n == 128) {
        if (R * a->tile_n + kV2Slots * R * 16 <= 512) tile_t = a->tile_n;
        else return fail(RNS_ERR_INVALID_ARGUMENT, "token tile %d leaves no tensor memory for the operand slots", a->tile_n);
    }
    gp.tile_t = tile_t;
    gp.opnd_col0 = R * tile_t;
    int cols = 32;
    while (cols < gp.opnd_col0 + kV2Slots * R * 16) cols <<= 1;
    gp.tmem_cols = cols;
    gp.plane_sub_bytes = (uint32_t)R * tile_t * kPackK;
    const int kblocks = (a->k + 63) / 64;
    const int npairs = (kblocks + 1) / 2;
    int stages = (227 * 1024 - 2048) / (int)(2 * gp.plane_sub_bytes);
    if (stages > kV2MaxPlaneStages) stages = kV2MaxPlaneStages;
    if (stages > npairs) stages = npairs;
    if (stages < 1) return fail(RNS_ERR_UNSUPPORTED, "token tile does not fit shared memory");
    gp.plane_stages = stages;
    gp.exact_residues = a->exact_residues ? 1 : 0;
    gp.active_ptr = a->d_active_channels;
    gp.planes = a->d_a_planes;
    gp.w = a->d_w;
    gp.w_npad = round_up_i64(a->n, kPackNPad);
    gp.out = a->d_out; gp.ldo = a->ldo; gp.out_type = a->out_type;
    gp.row_scale = a->d_row_scale; gp.row_scale_stride = a->row_scale_stride;
    gp.col_scale = a->d_col_scale; gp.bias = a->d_bias; gp.status = a->d_status;
    const dim3 grid((a->m + tile_t - 1) / tile_t, (a->n + 127) / 128, 1);
    if (grid.y > 65535) return fail(RNS_ERR_UNSUPPORTED, "too many feature tiles");
    const size_t smem = (size_t)stages * 2 * gp.plane_sub_bytes + 1024;
    switch (R) {
        case 2: return launch_tmem<2>(gp, grid, smem, st);
        case 3: return launch_tmem<3>(gp, grid, smem, st);
        case 4: return launch_tmem<4>(gp, grid, smem, st);
        case 5: return launch_tmem<5>(gp, grid, smem, st);
        default: return fail(RNS_ERR_UNSUPPORTED, "tensor-memory-operand kernel: 2..5 channels");
    }
}

}  // namespace rns

