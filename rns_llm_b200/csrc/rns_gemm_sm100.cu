// Fused RNS linear for sm_100a: TMA -> in-kernel residue encoding -> one
// tcgen05.mma.kind::i8 per residue channel (int32 accumulators in TMEM) ->
// epilogue with modular reduction, mixed-radix reconstruction, recentring and
// dequantisation.  One CTA computes one 128 x tile_n output tile; in PAIR mode two
// CTAs of a cluster (tcgen05 cta_group::2) compute a 256 x tile_n tile together:
// each holds its own 128 rows of A and HALF of the W tile, the leader CTA issues
// the MMAs, and each CTA's tensor memory receives its own 128 rows.  Pairing
// halves the W bytes every SM has to load, encode and feed to the tensor core.
//
// Warp roles (608 threads):
//   warp 0, 18  load producers (one elected lane each; even / odd K blocks)
//   warp 1      TMEM owner + MMA issuer (one elected lane)
//   warps 2..17 encoders during the K loop, epilogue afterwards
//
// Per pipeline stage the shared memory holds
//   raw  : source bytes as TMA delivers them (W tile, and the A tile when the
//          activations come as source integers), hardware-swizzled;
//   enc  : `channels` operand tiles for A and for W in the canonical K-major
//          swizzled layout the MMA reads.
// Residue encoding is elementwise, so an encoder thread reads 16 bytes at some
// offset of a raw tile and writes 16 bytes at the SAME offset of each channel's
// operand tile: the swizzle TMA applied is exactly the one the MMA expects.
//
// Every wait on an mbarrier is bounded in time; when one expires the CTA
// records RNS_ERR_DEVICE_TIMEOUT in the caller's status word, skips the
// remaining work, frees its tensor memory and returns.
#include "rns_common.cuh"
#include "rns_ptx.cuh"

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <atomic>
#include <mutex>
#include <type_traits>

namespace rns {

constexpr int kTileM = 128;
#ifndef RNS_WORKER_WARPS
#define RNS_WORKER_WARPS 16
#endif
constexpr int kWorkerWarps = RNS_WORKER_WARPS;
constexpr int kProducerWarpB = 2 + kWorkerWarps;          // second load producer
constexpr int kThreads = (3 + kWorkerWarps) * 32;
constexpr int kWorkerThreads = kWorkerWarps * 32;
constexpr int kMaxStages = 8;
#ifndef RNS_SPIN_WORKERS
#define RNS_SPIN_WORKERS 0
#endif
constexpr bool kSpinWorkers = RNS_SPIN_WORKERS != 0;   // worker warps poll without suspending

struct GemmParams {
    Plan plan;
    int32_t m, n, k;
    int32_t tile_n, tile_k;      // tile_k in {64,128}
    int32_t raw_stages;           // ring of raw (source byte) tiles: deep, covers the load latency
    int32_t enc_stages;           // ring of operand tiles written by the encoders: encode + MMA + release
    int32_t pl_stages;            // ring of activation planes (operands as loaded): load + MMA + release
    int32_t sub_blocks;           // K blocks of tile_k bytes per stage (one hand-over per stage:
                                  // a hand-over costs each role several hundred cycles of
                                  // dependent barrier operations, whatever the ring depth)
    uint32_t raw_sub_bytes, enc_sub_bytes;   // one K block inside a raw / an operand stage
    int32_t a_is_planes;
    int32_t a_packed, w_packed;   // operands in the packed tile layouts (bulk copies)
    const int8_t* a_ptr;          // packed activations / planes
    const int8_t* w_ptr;          // packed weights
    int64_t w_npad;               // padded weight rows of the packed layout
    int32_t tmem_cols;
    int32_t exact_residues;       // in-kernel encoder: exactly centred (1) or one-step reduced (0)
    int32_t enc_groups;           // worker warps are split into this many groups; group g encodes
                                  // the K blocks kb = g (mod groups), so that the fixed cost of a
                                  // stage hand-over overlaps with another group's encoding
    const int32_t* active_ptr;
    void* out;
    int64_t ldo;
    int32_t out_type;
    const float* row_scale;
    int32_t row_scale_stride;
    const float* col_scale;
    const float* bias;
    int32_t* status;
    int32_t* wait_info;
    // shared-memory map (byte offsets from the 1024-aligned base)
    uint32_t raw_stage_bytes, enc_stage_bytes, enc_ring_offset;   // raw ring first, operand ring after
    uint32_t pl_stage_bytes, pl_sub_bytes, pl_ring_offset;        // plane ring last (planes only)
    uint32_t off_raw_a, off_raw_w, off_enc_a, off_enc_w;          // inside a raw / an operand stage
    uint32_t tile_a_bytes, tile_w_bytes;
};

// Encodes the 16-byte chunks wt, wt+stride, ... of one raw tile into the R operand
// tiles.  ALL: every channel is active (no per-channel branch).  Up to four chunks
// are loaded before any is encoded, so that the shared-memory latency is paid once
// and the independent words give the scheduler something to overlap: a warp that
// works through one chunk at a time needs ~700 cycles per chunk, almost all of it
// dependent-issue latency.
#ifndef RNS_ENC_BATCH
#define RNS_ENC_BATCH 1
#endif
constexpr int kEncBatch = RNS_ENC_BATCH;

template <int R, bool FAST, bool ALL>
__device__ __forceinline__ void encode_chunks(const uint8_t* __restrict__ raw, uint8_t* __restrict__ enc,
                                              uint32_t tile_bytes, int chunks, int wt, int stride, int active,
                                              const uint32_t (&enc_hi)[R], const uint32_t (&enc_lo)[R],
                                              const uint32_t (&enc_mk)[R]) {
    for (int first = wt; first < chunks; first += kEncBatch * stride) {
        uint4 x[kEncBatch];
#pragma unroll
        for (int i = 0; i < kEncBatch; ++i) {
            const int ch = first + i * stride;
            if (ch < chunks) x[i] = *reinterpret_cast<const uint4*>(raw + ch * 16);
        }
#pragma unroll
        for (int i = 0; i < kEncBatch; ++i) {
            const int ch = first + i * stride;
            if (ch < chunks) {
                const uint32_t u0 = x[i].x ^ 0x80808080u, u1 = x[i].y ^ 0x80808080u;
                const uint32_t u2 = x[i].z ^ 0x80808080u, u3 = x[i].w ^ 0x80808080u;
                const uint32_t l0 = x[i].x & 0x7f7f7f7fu, l1 = x[i].y & 0x7f7f7f7fu;
                const uint32_t l2 = x[i].z & 0x7f7f7f7fu, l3 = x[i].w & 0x7f7f7f7fu;
                uint8_t* dst = enc + ch * 16;
#pragma unroll
                for (int c = 0; c < R; ++c) {
                    if (ALL || c < active) {
                        uint4 y;
                        y.x = encode_word<FAST>(u0, l0, enc_hi[c], enc_lo[c], enc_mk[c]);
                        y.y = encode_word<FAST>(u1, l1, enc_hi[c], enc_lo[c], enc_mk[c]);
                        y.z = encode_word<FAST>(u2, l2, enc_hi[c], enc_lo[c], enc_mk[c]);
                        y.w = encode_word<FAST>(u3, l3, enc_hi[c], enc_lo[c], enc_mk[c]);
                        *reinterpret_cast<uint4*>(dst + (size_t)c * tile_bytes) = y;
                    }
                }
            }
        }
    }
}

// Same, with the one-step reduced encoder (fold pattern shared by all channels).
template <int R, bool ALL>
__device__ __forceinline__ void encode_chunks_reduced(const uint8_t* __restrict__ raw, uint8_t* __restrict__ enc,
                                                      uint32_t tile_bytes, int chunks, int wt, int stride,
                                                      int active, const uint32_t (&mfold)[R]) {
    for (int first = wt; first < chunks; first += kEncBatch * stride) {
        uint4 x[kEncBatch];
#pragma unroll
        for (int i = 0; i < kEncBatch; ++i) {
            const int ch = first + i * stride;
            if (ch < chunks) x[i] = *reinterpret_cast<const uint4*>(raw + ch * 16);
        }
#pragma unroll
        for (int i = 0; i < kEncBatch; ++i) {
            const int ch = first + i * stride;
            if (ch < chunks) {
                const uint32_t u0 = x[i].x ^ 0x80808080u, u1 = x[i].y ^ 0x80808080u;
                const uint32_t u2 = x[i].z ^ 0x80808080u, u3 = x[i].w ^ 0x80808080u;
                const uint32_t d0 = fold_pattern(x[i].x), d1 = fold_pattern(x[i].y);
                const uint32_t d2 = fold_pattern(x[i].z), d3 = fold_pattern(x[i].w);
                uint8_t* dst = enc + ch * 16;
#pragma unroll
                for (int c = 0; c < R; ++c) {
                    if (ALL || c < active) {
                        uint4 y;
                        y.x = encode_word_reduced(u0, d0, mfold[c]);
                        y.y = encode_word_reduced(u1, d1, mfold[c]);
                        y.z = encode_word_reduced(u2, d2, mfold[c]);
                        y.w = encode_word_reduced(u3, d3, mfold[c]);
                        *reinterpret_cast<uint4*>(dst + (size_t)c * tile_bytes) = y;
                    }
                }
            }
        }
    }
}

// Slot and round of consecutive stages in a ring, kept incrementally: a division by a
// run-time ring depth costs a role ~150 cycles of dependent latency, several times per
// stage and on every role's critical path.
struct RingPos {
    int slot;
    uint32_t round;
    int depth;
    __device__ RingPos(int depth_, int start) : slot(start % depth_), round((uint32_t)(start / depth_)), depth(depth_) {}
    __device__ void advance(int by) {
        slot += by;
        while (slot >= depth) { slot -= depth; ++round; }
    }
};

struct __align__(8) SharedCtl {
    uint64_t full_raw[kMaxStages];    // raw tiles of the stage have landed
    uint64_t empty_raw[kMaxStages];   // encoders have read the raw tiles
    uint64_t full_enc[kMaxStages];
    uint64_t empty_enc[kMaxStages];
    uint64_t full_pl[kMaxStages];     // activation planes of the stage have landed
    uint64_t empty_pl[kMaxStages];    // ... and the MMAs that read them are done
    uint64_t acc_full;
    uint64_t peer_ready[kMaxStages];  // PAIR, leader only: the peer CTA's stage is complete
    uint32_t tmem_base;
    int abort;
};

// J_/ES_/PS_/RS_ > 0 select the "fixed" instantiation: K blocks per stage and the depths
// of the operand, plane and raw rings are compile-time constants, and so is everything
// that follows from the hot configuration they stand for (packed planes and packed
// weights, 64-byte K blocks, every channel active, one-step reduced residues, G_
// encoder groups, tile_n = 128 up to four channels and 96 for five).  The roles' loops
// are chains of dependent scalar instructions, a few cycles each: every run-time
// parameter folded into a constant shortens a stage.  All zeros: everything run-time.
template <int R, bool PAIR, int J_, int ES_, int PS_, int RS_, int G_>
__global__ void __launch_bounds__(kThreads, 1)
rns_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                const __grid_constant__ GemmParams p) {
    extern __shared__ uint8_t smem_dyn[];
    __shared__ SharedCtl ctl;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t tiles_base = (smem_addr(smem_dyn) + 1023u) & ~1023u;
    uint8_t* tiles_ptr = smem_dyn + (tiles_base - smem_addr(smem_dyn));

    // Grid: x walks the column tiles fastest, so that CTAs resident at the same time
    // share their A tiles in L2.  PAIR: x = 2 * column tile + rank (the two CTAs of a
    // cluster are neighbours in x), y = pair of row tiles; rank 0 leads.  Each CTA of
    // a pair loads and encodes tile_n/2 rows of W starting at w_row0.
    const uint32_t pair_rank = PAIR ? cluster_cta_rank() : 0u;
    constexpr bool FIXED = J_ > 0;
    // RS_ < 0: no raw ring at all; the encoder threads read their weight bytes from
    // global memory into registers, two of their stages ahead (packed weights, J_ == 1).
    constexpr bool W_DIRECT = FIXED && RS_ < 0;
    // ... and with PS_ == 0 the same goes for the activations: they arrive as packed int8
    // (one byte per value instead of R planes), the encoder threads produce the operand
    // tiles of both sides, and the main loop has no bulk copies at all.
    constexpr bool A_DIRECT = W_DIRECT && PS_ == 0;
    // The operand slot and the plane slot of a stage are released by the same MMAs.
    // When the operand ring is at least as deep as the plane ring, one commit per
    // stage serves both: the plane producer of stage st waits on the operand ring's
    // barrier of stage st - PS_ (one commit less on the MMA warp's path).
    constexpr bool ONE_COMMIT = W_DIRECT && !PAIR && ES_ >= PS_;
    // In those kernels warp 0 has no loads to issue and becomes a second MMA issuer:
    // warp 1 takes the even stages, warp 0 the odd ones.  Integer accumulation does not
    // depend on the order of the MMAs; the accumulators are zeroed beforehand, so that
    // no MMA has to come first.  Each issuer's instruction stream per stage is longer
    // than the MMAs it issues; two of them keep the tensor pipe fed.
    // Only with an even operand-ring depth: a warp that takes every other stage then always
    // meets the same slots and sees every phase of their barriers.  With an odd depth it
    // would skip alternate phases of a slot, and a parity wait cannot tell "the phase before
    // last has completed" from the awaited one: when the planes of stage s landed after
    // those of stage s + 1, the issuer of stage s + 3 could pass its wait early.
    constexpr bool TWO_ISSUERS = ONE_COMMIT && (ES_ % 2 == 0);
    const int tile_k = FIXED ? 64 : p.tile_k;
    const int tile_n = FIXED ? (R <= 4 ? 128 : 96) : p.tile_n;
    const int m_tile = PAIR ? 2 * (int)blockIdx.y + (int)pair_rank : (int)blockIdx.y;
    const int n0 = (PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x) * tile_n;
    const int w_rows = PAIR ? tile_n / 2 : tile_n;
    const int w_row0 = n0 + (int)pair_rank * w_rows;
    const int m0 = m_tile * kTileM;
    const int kblocks = (p.k + tile_k - 1) / tile_k;
    const int raw_stages = FIXED ? (RS_ > 0 ? RS_ : 1) : p.raw_stages, enc_stages = FIXED ? ES_ : p.enc_stages;
    const int J = FIXED ? J_ : p.sub_blocks;          // K blocks per stage
    const int nstages = (kblocks + J - 1) / J;       // stage hand-overs in the K loop
    const bool a_planes = FIXED ? !A_DIRECT : p.a_is_planes != 0;
    const bool a_packed = FIXED ? true : p.a_packed != 0, w_packed = FIXED ? true : p.w_packed != 0;
    const int groups = FIXED ? G_ : p.enc_groups;
    // Shared-memory map: the parameters' values, or the same values as constants.
    const uint32_t tile_a_bytes = FIXED ? (uint32_t)(kTileM * 64) : p.tile_a_bytes;
    const uint32_t tile_w_bytes = FIXED ? (uint32_t)((PAIR ? tile_n / 2 : tile_n) * 64) : p.tile_w_bytes;
    const uint32_t raw_sub_bytes = FIXED ? ((tile_w_bytes + 1023u) & ~1023u) : p.raw_sub_bytes;
    const uint32_t enc_sub_bytes = FIXED ? (((uint32_t)R * (tile_w_bytes + (A_DIRECT ? tile_a_bytes : 0u)) + 1023u) & ~1023u) : p.enc_sub_bytes;
    const uint32_t pl_sub_bytes = FIXED ? (uint32_t)R * tile_a_bytes : p.pl_sub_bytes;
    const uint32_t raw_stage_bytes = FIXED ? (uint32_t)J_ * raw_sub_bytes : p.raw_stage_bytes;
    const uint32_t enc_stage_bytes = FIXED ? (uint32_t)J_ * enc_sub_bytes : p.enc_stage_bytes;
    const uint32_t pl_stage_bytes = FIXED ? (uint32_t)J_ * pl_sub_bytes : p.pl_stage_bytes;
    const uint32_t enc_ring_offset = FIXED ? (uint32_t)(RS_ > 0 ? RS_ : 0) * raw_stage_bytes : p.enc_ring_offset;
    const uint32_t pl_ring_offset = FIXED ? enc_ring_offset + (uint32_t)ES_ * enc_stage_bytes : p.pl_ring_offset;
    const uint32_t off_raw_w = FIXED ? 0u : p.off_raw_w, off_raw_a = FIXED ? tile_w_bytes : p.off_raw_a;
    const uint32_t off_enc_a = FIXED ? 0u : p.off_enc_a, off_enc_w = FIXED ? (A_DIRECT ? (uint32_t)R * tile_a_bytes : 0u) : p.off_enc_w;

    int active = R;
    if (!FIXED && p.active_ptr != nullptr) {
        active = *p.active_ptr;
        active = active < 1 ? 1 : (active > R ? R : active);
    }

    if (threadIdx.x == 0) {
        ctl.abort = 0;
        for (int s = 0; s < kMaxStages; ++s) {
            mbar_init(smem_addr(&ctl.full_raw[s]), 1);
            mbar_init(smem_addr(&ctl.empty_raw[s]), kWorkerWarps / groups);
            // ONE_COMMIT kernels: the plane load of a stage signals the operand ring's
            // "full" barrier too (one more arrival), so the MMA warp waits once per stage.
            mbar_init(smem_addr(&ctl.full_enc[s]), kWorkerWarps / groups + ((ONE_COMMIT && !A_DIRECT) ? 1 : 0));
            mbar_init(smem_addr(&ctl.empty_enc[s]), 1);
            mbar_init(smem_addr(&ctl.full_pl[s]), 1);
            mbar_init(smem_addr(&ctl.empty_pl[s]), 1);
            mbar_init(smem_addr(&ctl.peer_ready[s]), 1);
        }
        mbar_init(smem_addr(&ctl.acc_full), TWO_ISSUERS ? 2 : 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        if (PAIR) {
            tmem_alloc2(smem_addr(&ctl.tmem_base), (uint32_t)p.tmem_cols);
            tmem_relinquish2();
        } else {
            tmem_alloc(smem_addr(&ctl.tmem_base), (uint32_t)p.tmem_cols);
            tmem_relinquish();
        }
    }
    tc_fence_before();
    // Barriers of both CTAs must exist before the partner signals them.
    if (PAIR) cluster_sync_all(); else __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = ctl.tmem_base;
    volatile int* abort = &ctl.abort;
    const uint32_t enc_base = tiles_base + enc_ring_offset;
    const uint32_t pl_base = tiles_base + pl_ring_offset;
    const int pl_stages = FIXED ? (PS_ > 0 ? PS_ : 1) : p.pl_stages;

    if (warp == 0 && !TWO_ISSUERS) {
        // ------------------------------ raw-tile producer -------------------------
        // Source bytes (the W tile, and the A tile when activations are not planes)
        // go to the deep raw ring; a slot is free as soon as the encoders have read it.
        if (lane == 0 && !W_DIRECT) {
            const uint32_t tx = tile_w_bytes +
                                (a_planes ? 0u : tile_a_bytes);
            RingPos ring(raw_stages, 0);
            for (int st = 0; st < nstages; ++st, ring.advance(1)) {
                const int s = ring.slot;
                const uint32_t round = ring.round;
                const uint32_t stage = tiles_base + (uint32_t)s * raw_stage_bytes;
                const int jn = (FIXED && J_ == 1) ? 1 : min(J, kblocks - st * J);
                if (round > 0 && !wait_bounded<false, true>(smem_addr(&ctl.empty_raw[s]), (round - 1) & 1, abort, wait_code(1, st))) break;
                const uint32_t fr = smem_addr(&ctl.full_raw[s]);
                mbar_arrive_expect_tx(fr, tx * (uint32_t)jn);
                for (int j = 0; j < jn; ++j) {
                    const int kb = st * J + j;
                    const uint32_t sub = stage + (uint32_t)j * raw_sub_bytes;
                    if (w_packed)
                        bulk_load(sub + off_raw_w,
                                  p.w_ptr + ((int64_t)kb * p.w_npad + w_row0) * kPackK, tile_w_bytes, fr);
                    else
                        tma_load_2d(sub + off_raw_w, &map_w, fr, kb * tile_k, w_row0);
                    if (!a_planes) {
                        const int64_t a_tile = (int64_t)m_tile * kblocks + kb;   // packed tile index
                        if (a_packed)
                            bulk_load(sub + off_raw_a, p.a_ptr + a_tile * (kPackM * kPackK), tile_a_bytes, fr);
                        else
                            tma_load_2d(sub + off_raw_a, &map_a, fr, kb * tile_k, m0);
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == kProducerWarpB) {
        // ------------------------------ plane producer ----------------------------
        // Activation planes are MMA operands as they arrive: they go to a ring of
        // their own, deep enough to cover the load latency, whose slots the MMAs release.
        if (lane == 0 && a_planes) {
            const uint32_t a_bytes = (uint32_t)active * tile_a_bytes;
            RingPos ring(pl_stages, 0);
            RingPos released(enc_stages, 0);   // ONE_COMMIT: the stage whose plane slot is reused
            RingPos filled(enc_stages, 0);     // ONE_COMMIT: operand-ring barrier of the stage being loaded
            for (int st = 0; st < nstages; ++st, ring.advance(1)) {
                const int s = ring.slot;
                const uint32_t round = ring.round;
                const uint32_t stage = pl_base + (uint32_t)s * pl_stage_bytes;
                const int jn = (FIXED && J_ == 1) ? 1 : min(J, kblocks - st * J);
                if (ONE_COMMIT) {
                    if (st >= pl_stages) {
                        if (!wait_bounded<false, true>(smem_addr(&ctl.empty_enc[released.slot]), released.round & 1, abort, wait_code(2, st))) break;
                        released.advance(1);
                    }
                } else if (round > 0 && !wait_bounded<false, true>(smem_addr(&ctl.empty_pl[s]), (round - 1) & 1, abort, wait_code(2, st))) break;
                const uint32_t fp = ONE_COMMIT ? smem_addr(&ctl.full_enc[filled.slot]) : smem_addr(&ctl.full_pl[s]);
                if (ONE_COMMIT) filled.advance(1);
                mbar_arrive_expect_tx(fp, a_bytes * (uint32_t)jn);
                for (int j = 0; j < jn; ++j) {
                    const int kb = st * J + j;
                    const uint32_t sub = stage + (uint32_t)j * pl_sub_bytes;
                    const int64_t a_tile = (int64_t)m_tile * kblocks + kb;
                    if (a_packed) {
                        bulk_load(sub, p.a_ptr + a_tile * ((int64_t)R * kPackM * kPackK), a_bytes, fp);
                    } else {
                        for (int c = 0; c < active; ++c)
                            tma_load_3d(sub + (uint32_t)c * tile_a_bytes, &map_a, fp, kb * tile_k, m0, c);
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1 || (TWO_ISSUERS && warp == 0)) {
        // ------------------------------ MMA issuer --------------------------------
        // PAIR: only the leader issues MMAs; the peer's lane relays "my stage is
        // complete" to the leader's peer_ready barrier.  Completion of the MMAs is
        // signalled to the empty_enc / acc_full barriers of both CTAs.
        if (lane == 0 && PAIR && pair_rank != 0) {
            RingPos ring(enc_stages, 0), ring_pl(pl_stages, 0);
            for (int st = 0; st < nstages; ++st, ring.advance(1), ring_pl.advance(1)) {
                const int s = ring.slot;
                const uint32_t round = ring.round;
                if (!wait_bounded<false, true>(smem_addr(&ctl.full_enc[s]), round & 1, abort, wait_code(3, st))) break;
                if (a_planes && !wait_bounded<false, true>(smem_addr(&ctl.full_pl[ring_pl.slot]),
                                                           ring_pl.round & 1, abort, wait_code(4, st))) break;
                mbar_arrive_remote(smem_addr(&ctl.peer_ready[s]), 0);
            }
        } else if (!PAIR || pair_rank == 0) {
            // The whole warp runs this loop, so that the addresses and descriptors
            // below are warp-uniform values (computed once, in the uniform datapath);
            // one elected lane issues the MMAs and the commits.  Issued from inside a
            // single-lane branch the same arithmetic costs ~190 cycles per MMA, three
            // times the MMA's own duration.
            const uint32_t idesc = make_idesc(PAIR ? 256u : 128u, (uint32_t)tile_n);
            const uint64_t desc0 = make_smem_desc(0, tile_k);        // everything but the address
            const uint32_t a_lo0 = (a_planes ? pl_base : enc_base + off_enc_a) >> 4, w_lo0 = (enc_base + off_enc_w) >> 4;
            const uint32_t stage_step = enc_stage_bytes >> 4, sub_step = enc_sub_bytes >> 4;
            const uint32_t a_stage_step = (a_planes ? pl_stage_bytes : enc_stage_bytes) >> 4;
            const uint32_t a_sub_step = (a_planes ? pl_sub_bytes : enc_sub_bytes) >> 4;
            const uint32_t a_step = tile_a_bytes >> 4, w_step = tile_w_bytes >> 4;
            const int nks = tile_k / 32;
            const int mma_channels = active;
            uint32_t a_off[R], w_off[R];
#pragma unroll
            for (int c = 0; c < R; ++c) { a_off[c] = (uint32_t)c * a_step; w_off[c] = (uint32_t)c * w_step; }
            bool ok = true;
            const int st_first = (TWO_ISSUERS && warp == 0) ? 1 : 0, st_step = TWO_ISSUERS ? 2 : 1;
            RingPos ring(enc_stages, st_first), ring_pl(pl_stages, st_first);
            for (int st = st_first; st < nstages && ok; st += st_step, ring.advance(st_step), ring_pl.advance(st_step)) {
                const int s = ring.slot;
                const uint32_t round = ring.round;
                const int jn = (FIXED && J_ == 1) ? 1 : min(J, kblocks - st * J);
                const int sa = a_planes ? ring_pl.slot : s;       // slot of the A operands
                ok = warp_wait_bounded<false, true>(smem_addr(&ctl.full_enc[s]), round & 1, abort, wait_code(5, st));
                if (ok && a_planes && !ONE_COMMIT)
                    ok = warp_wait_bounded<false, true>(smem_addr(&ctl.full_pl[sa]), ring_pl.round & 1, abort, wait_code(6, st));
                if (ok && PAIR) ok = warp_wait_bounded<true>(smem_addr(&ctl.peer_ready[s]), round & 1, abort, wait_code(7, st));
                if (!ok) break;
                tc_fence_after();
                const uint32_t a_st = a_lo0 + (uint32_t)sa * a_stage_step, w_st = w_lo0 + (uint32_t)s * stage_step;
                const uint32_t empty_bar = smem_addr(&ctl.empty_enc[s]);
                const uint32_t empty_pl_bar = smem_addr(&ctl.empty_pl[sa]);
                for (int j = 0; j < jn; ++j) {
                    const uint32_t a_j = a_st + (uint32_t)j * a_sub_step, w_j = w_st + (uint32_t)j * sub_step;
                    const uint32_t first = (TWO_ISSUERS || st > 0 || j > 0) ? 1u : 0u;
                    if (elect_one()) {
#pragma unroll
                        for (int c = 0; c < R; ++c) {
                            if (c < mma_channels) {
                                const uint32_t d = tmem_base + (uint32_t)(c * tile_n);
#pragma unroll
                                for (int ks = 0; ks < 4; ++ks) {
                                    if (ks < nks) {
                                        const uint64_t da = desc0 | (uint64_t)(a_j + a_off[c] + (uint32_t)ks * 2u);
                                        const uint64_t db = desc0 | (uint64_t)(w_j + w_off[c] + (uint32_t)ks * 2u);
                                        const uint32_t acc = ks > 0 ? 1u : first;
                                        if (PAIR) umma_i8_pair(d, da, db, idesc, acc);
                                        else umma_i8(d, da, db, idesc, acc);
                                    }
                                }
                            }
                        }
                    }
                    __syncwarp();
                }
                if (elect_one()) {
                    if (PAIR) umma_commit_pair(empty_bar);
                    else umma_commit(empty_bar);
                    if (a_planes && !ONE_COMMIT) {
                        if (PAIR) umma_commit_pair(empty_pl_bar);
                        else umma_commit(empty_pl_bar);
                    }
                }
                __syncwarp();
            }
            if (ok && elect_one()) {
                if (PAIR) umma_commit_pair(smem_addr(&ctl.acc_full));
                else umma_commit(smem_addr(&ctl.acc_full));
            }
        }
        __syncwarp();
    } else {
        // ------------------------------ encoders ----------------------------------
        const int group = (warp - 2) % groups;
        const int group_threads = kWorkerThreads / groups;
        const int wt = ((warp - 2) / groups) * 32 + lane;   // index inside the group
        const int rows_a = min(kTileM, p.m - m0);
        const int rows_w = max(0, min(w_rows, p.n - w_row0));
        // 16-byte chunks that hold valid rows (row r occupies bytes [r*tile_k, (r+1)*tile_k)
        // of a tile in every swizzle mode).
        const int chunks_a = a_planes ? 0 : rows_a * (tile_k / 16);
        const int chunks_w = rows_w * (tile_k / 16);
        uint32_t enc_hi[R], enc_lo[R], enc_mk[R], enc_mfold[R];
#pragma unroll
        for (int c = 0; c < R; ++c) {
            enc_hi[c] = p.plan.enc_hi[c]; enc_lo[c] = p.plan.enc_lo[c]; enc_mk[c] = p.plan.enc_mk[c];
            enc_mfold[c] = p.plan.enc_mfold[c];
        }
        const bool reduced = FIXED ? true : p.exact_residues == 0;
        const bool fast = p.plan.encode_fast != 0;
        bool ok = true;
        if constexpr (TWO_ISSUERS) {
            // Zero the accumulators (this warp's lane quarter, 128 of the 512 columns):
            // with two issuers no MMA is "the first one" that would overwrite them.
            const uint32_t zero_at = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(((warp - 2) >> 2) * 128);
            uint32_t zeros[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) zeros[i] = 0u;
#pragma unroll
            for (int i = 0; i < 8; ++i) tmem_st16(zero_at + (uint32_t)(i * 16), zeros);
            tmem_st_wait();
            tc_fence_before();
        }
        if constexpr (W_DIRECT) {
            // Chunks wt, wt + group_threads, ... of the W tile of K block kb sit at
            // w_tile(kb) + 16 * chunk in the packed weight matrix (a tile is contiguous).
            // Two of this group's stages are kept in registers ahead of the one encoded.
            constexpr int kGroupThreads = kWorkerThreads / (G_ > 0 ? G_ : 1);
            constexpr int kChunks = ((R <= 4 ? 128 : 96) * 4 + kGroupThreads - 1) / kGroupThreads;   // per thread and K block
            const int8_t* w_tile0 = p.w_ptr + (int64_t)w_row0 * kPackK + (int64_t)wt * 16;
            const int64_t kb_stride = p.w_npad * kPackK;
            // A_DIRECT: likewise for the activation tile (128 rows, contiguous 8 KB per K block).
            constexpr int kChunksA = A_DIRECT ? (kTileM * 4 + kGroupThreads - 1) / kGroupThreads : 1;
            const int8_t* a_tile0 = p.a_ptr + (int64_t)m_tile * kblocks * (kPackM * kPackK) + (int64_t)wt * 16;
            uint4 cur_a[kChunksA], nxt_a[kChunksA];
            auto load_stage_a = [&](int st, uint4 (&dst)[kChunksA]) {
#pragma unroll
                for (int i = 0; i < kChunksA; ++i) {
                    const int ch = wt + i * group_threads;
                    if (A_DIRECT && st < nstages && ch < chunks_a)
                        dst[i] = __ldg(reinterpret_cast<const uint4*>(a_tile0 + (int64_t)st * (kPackM * kPackK) + (int64_t)i * group_threads * 16));
                    else
                        dst[i] = make_uint4(0u, 0u, 0u, 0u);
                }
            };
            auto encode_chunk = [&](const uint4 x, uint8_t* dst, uint32_t tile_bytes) {
                const uint32_t u0 = x.x ^ 0x80808080u, u1 = x.y ^ 0x80808080u;
                const uint32_t u2 = x.z ^ 0x80808080u, u3 = x.w ^ 0x80808080u;
                const uint32_t d0 = fold_pattern(x.x), d1 = fold_pattern(x.y);
                const uint32_t d2 = fold_pattern(x.z), d3 = fold_pattern(x.w);
#pragma unroll
                for (int c = 0; c < R; ++c) {
                    uint4 y;
                    y.x = encode_word_reduced(u0, d0, enc_mfold[c]);
                    y.y = encode_word_reduced(u1, d1, enc_mfold[c]);
                    y.z = encode_word_reduced(u2, d2, enc_mfold[c]);
                    y.w = encode_word_reduced(u3, d3, enc_mfold[c]);
                    *reinterpret_cast<uint4*>(dst + (size_t)c * tile_bytes) = y;
                }
            };
            if (A_DIRECT) { load_stage_a(group, cur_a); load_stage_a(group + groups, nxt_a); }
            uint4 cur[kChunks], nxt[kChunks];
            auto load_stage = [&](int st, uint4 (&dst)[kChunks]) {
#pragma unroll
                for (int i = 0; i < kChunks; ++i) {
                    const int ch = wt + i * group_threads;
                    if (st < nstages && ch < chunks_w)
                        dst[i] = __ldg(reinterpret_cast<const uint4*>(w_tile0 + (int64_t)st * kb_stride + (int64_t)i * group_threads * 16));
                    else
                        dst[i] = make_uint4(0u, 0u, 0u, 0u);
                }
            };
            load_stage(group, cur);
            load_stage(group + groups, nxt);
            RingPos ring_e(enc_stages, group);
            for (int st = group; st < nstages && ok; st += groups, ring_e.advance(groups)) {
                const int se = ring_e.slot;
                uint8_t* enc = tiles_ptr + enc_ring_offset + (size_t)se * enc_stage_bytes;
                uint4 ahead[kChunks];
                load_stage(st + 2 * groups, ahead);
                uint4 ahead_a[kChunksA];
                if (A_DIRECT) load_stage_a(st + 2 * groups, ahead_a);
                if (ring_e.round > 0)
                    ok = warp_wait_bounded<false, kSpinWorkers>(smem_addr(&ctl.empty_enc[se]), (ring_e.round - 1) & 1, abort, wait_code(8, st));
                if (!ok) break;
#pragma unroll
                for (int i = 0; i < kChunks; ++i) {
                    const int ch = wt + i * group_threads;
                    if (ch < chunks_w) encode_chunk(cur[i], enc + off_enc_w + ch * 16, tile_w_bytes);
                }
                if (A_DIRECT) {
#pragma unroll
                    for (int i = 0; i < kChunksA; ++i) {
                        const int ch = wt + i * group_threads;
                        if (ch < chunks_a) encode_chunk(cur_a[i], enc + off_enc_a + ch * 16, tile_a_bytes);
                    }
#pragma unroll
                    for (int i = 0; i < kChunksA; ++i) { cur_a[i] = nxt_a[i]; nxt_a[i] = ahead_a[i]; }
                }
#pragma unroll
                for (int i = 0; i < kChunks; ++i) { cur[i] = nxt[i]; nxt[i] = ahead[i]; }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_addr(&ctl.full_enc[se]));
            }
        }
        RingPos ring_r(raw_stages, group), ring_e(enc_stages, group);
        for (int st = group; st < nstages && ok && !W_DIRECT; st += groups, ring_r.advance(groups), ring_e.advance(groups)) {
            const int sr = ring_r.slot, se = ring_e.slot;
            const uint32_t round_r = ring_r.round, round_e = ring_e.round;
            const uint8_t* raw_stage = tiles_ptr + (size_t)sr * raw_stage_bytes;
            uint8_t* enc_stage = tiles_ptr + enc_ring_offset + (size_t)se * enc_stage_bytes;
            const int jn = (FIXED && J_ == 1) ? 1 : min(J, kblocks - st * J);
            // Order matters once several groups run ahead of each other: the operand
            // slot must first be released by the MMAs of its previous revolution of the ring.  Because
            // the raw ring is at least as deep as the operand ring, that also proves
            // that the raw slot's previous revolution has completed, which makes the parity
            // of the full_raw wait unambiguous.
            if (round_e > 0) ok = warp_wait_bounded<false, kSpinWorkers>(smem_addr(&ctl.empty_enc[se]), (round_e - 1) & 1, abort, wait_code(9, st));
            if (ok) ok = warp_wait_bounded<false, kSpinWorkers>(smem_addr(&ctl.full_raw[sr]), round_r & 1, abort, wait_code(10, st));
            if (!ok) break;
            // part 0: the W tile; part 1: the A tile (nothing to do when activations are planes)
            const int parts = (FIXED || a_planes) ? 1 : 2;
            for (int jp = 0; jp < parts * jn; ++jp) {
                const int j = parts == 1 ? jp : jp >> 1, part = parts == 1 ? 0 : jp & 1;
                const int chunks = part == 0 ? chunks_w : chunks_a;
                const uint8_t* raw = raw_stage + (size_t)j * raw_sub_bytes + (part == 0 ? off_raw_w : off_raw_a);
                uint8_t* enc = enc_stage + (size_t)j * enc_sub_bytes + (part == 0 ? off_enc_w : off_enc_a);
                const uint32_t tile_bytes = part == 0 ? tile_w_bytes : tile_a_bytes;
                if (reduced && active == R)
                    encode_chunks_reduced<R, true>(raw, enc, tile_bytes, chunks, wt, group_threads, active, enc_mfold);
                else if (reduced)
                    encode_chunks_reduced<R, false>(raw, enc, tile_bytes, chunks, wt, group_threads, active, enc_mfold);
                else if (fast && active == R)
                    encode_chunks<R, true, true>(raw, enc, tile_bytes, chunks, wt, group_threads, active, enc_hi, enc_lo, enc_mk);
                else if (fast)
                    encode_chunks<R, true, false>(raw, enc, tile_bytes, chunks, wt, group_threads, active, enc_hi, enc_lo, enc_mk);
                else
                    encode_chunks<R, false, false>(raw, enc, tile_bytes, chunks, wt, group_threads, active, enc_hi, enc_lo, enc_mk);
            }
            // Every writer makes its stores visible to the async proxy, the warp
            // converges, and one lane signals for the warp (arrivals on one mbarrier
            // serialise): the operand tiles are ready, the raw slot may be refilled.
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(smem_addr(&ctl.full_enc[se]));
                mbar_arrive(smem_addr(&ctl.empty_raw[sr]));
            }
        }

        // ------------------------------ epilogue ----------------------------------
        if (ok) ok = warp_wait_bounded(smem_addr(&ctl.acc_full), 0, abort, wait_code(11, 0));
        if (ok) {
            tc_fence_after();
            const int quarter = warp & 3;             // TMEM lanes 32*quarter .. +31
            const int part = (warp - 2) >> 2;         // 8-column chunks are dealt round-robin
            const int row = m0 + quarter * 32 + lane;
            const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
            float rs = 0.0f;
            const bool is_float = p.out_type >= RNS_OUT_F16;
            if (is_float && row < p.m) rs = p.row_scale[(int64_t)row * p.row_scale_stride];
            using XInt = typename std::conditional<(R <= 4), int, long long>::type;
            // load: R x 8 accumulator columns of this thread's row (warp-collective);
            // finish: reconstruction, dequantisation and the store of those 8 outputs.
            auto load = [&](int col, int (&acc)[R][8]) {
                __syncwarp();
#pragma unroll
                for (int c = 0; c < R; ++c) {
                    if (c < active) {
                        tmem_ld8(lane_base + (uint32_t)(c * tile_n + col), acc[c]);
                    } else {
#pragma unroll
                        for (int e = 0; e < 8; ++e) acc[c][e] = 0;
                    }
                }
            };
            auto finish = [&](int col, const int (&acc)[R][8]) {
                const int gcol = n0 + col;
                if (row >= p.m || gcol >= p.n) return;
                XInt xs[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    int one[R];
#pragma unroll
                    for (int c = 0; c < R; ++c) one[c] = acc[c][e];
                    if constexpr (R <= 4) xs[e] = reconstruct32<R>(one, p.plan, active);
                    else xs[e] = reconstruct<R>(one, p.plan, active);
                }
                const int valid = min(8, p.n - gcol);
                const int64_t o = (int64_t)row * p.ldo + gcol;
                if (p.out_type == RNS_OUT_INT64) {
                    long long* out = static_cast<long long*>(p.out) + o;
#pragma unroll
                    for (int e = 0; e < 8; ++e) if (e < valid) out[e] = xs[e];
                } else if (p.out_type == RNS_OUT_INT32) {
                    int* out = static_cast<int*>(p.out) + o;
#pragma unroll
                    for (int e = 0; e < 8; ++e) if (e < valid) out[e] = (int)xs[e];
                } else {
                    // column scales and bias of these 8 outputs: two 16-byte loads each when
                    // the group is whole and aligned
                    float cs[8], bs[8];
                    const float* cs_ptr = p.col_scale + gcol;
                    const float* bs_ptr = p.bias != nullptr ? p.bias + gcol : nullptr;
                    const bool whole = valid == 8 && (reinterpret_cast<uintptr_t>(cs_ptr) & 15) == 0 &&
                                       (reinterpret_cast<uintptr_t>(bs_ptr) & 15) == 0;
                    if (whole) {
                        const float4 c0 = __ldg(reinterpret_cast<const float4*>(cs_ptr));
                        const float4 c1 = __ldg(reinterpret_cast<const float4*>(cs_ptr) + 1);
                        cs[0] = c0.x; cs[1] = c0.y; cs[2] = c0.z; cs[3] = c0.w;
                        cs[4] = c1.x; cs[5] = c1.y; cs[6] = c1.z; cs[7] = c1.w;
                        if (bs_ptr != nullptr) {
                            const float4 b0 = __ldg(reinterpret_cast<const float4*>(bs_ptr));
                            const float4 b1 = __ldg(reinterpret_cast<const float4*>(bs_ptr) + 1);
                            bs[0] = b0.x; bs[1] = b0.y; bs[2] = b0.z; bs[3] = b0.w;
                            bs[4] = b1.x; bs[5] = b1.y; bs[6] = b1.z; bs[7] = b1.w;
                        }
                    } else {
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            cs[e] = e < valid ? cs_ptr[e] : 0.0f;
                            bs[e] = (e < valid && bs_ptr != nullptr) ? bs_ptr[e] : 0.0f;
                        }
                    }
                    float y[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        float xf;
                        if constexpr (R <= 4) xf = __int2float_rn(xs[e]);
                        else xf = __ll2float_rn(xs[e]);
                        float v = __fmul_rn(__fmul_rn(xf, rs), cs[e]);
                        if (bs_ptr != nullptr) v = __fadd_rn(v, bs[e]);
                        y[e] = v;
                    }
                    if (p.out_type == RNS_OUT_F32) {
                        float* out = static_cast<float*>(p.out) + o;
#pragma unroll
                        for (int e = 0; e < 8; ++e) if (e < valid) out[e] = y[e];
                    } else if (p.out_type == RNS_OUT_F16) {
                        __half* out = static_cast<__half*>(p.out) + o;
                        if (valid == 8 && ((reinterpret_cast<uintptr_t>(out) & 15) == 0)) {
                            __half2 h[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e) h[e] = __floats2half2_rn(y[2 * e], y[2 * e + 1]);
                            *reinterpret_cast<uint4*>(out) = *reinterpret_cast<const uint4*>(h);
                        } else {
#pragma unroll
                            for (int e = 0; e < 8; ++e) if (e < valid) out[e] = __float2half_rn(y[e]);
                        }
                    } else {
                        __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.out) + o;
                        if (valid == 8 && ((reinterpret_cast<uintptr_t>(out) & 15) == 0)) {
                            __nv_bfloat162 h[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e) h[e] = __floats2bfloat162_rn(y[2 * e], y[2 * e + 1]);
                            *reinterpret_cast<uint4*>(out) = *reinterpret_cast<const uint4*>(h);
                        } else {
#pragma unroll
                            for (int e = 0; e < 8; ++e) if (e < valid) out[e] = __float2bfloat16_rn(y[e]);
                        }
                    }
                }
            };
            constexpr int kColStep = (kWorkerWarps / 4) * 8;
            if constexpr (FIXED && R <= 4) {
                // The loads of the next column group are in flight while this one is
                // finished (two register buffers, loop unrolled by hand).
                constexpr int kIters = (R <= 4 ? 128 : 96) / kColStep;
                const int col0 = part * 8;
                int a0[R][8], a1[R][8];
                load(col0, a0);
#pragma unroll
                for (int it = 0; it < kIters; it += 2) {
                    tmem_ld_wait();
                    if (it + 1 < kIters) load(col0 + (it + 1) * kColStep, a1);
                    finish(col0 + it * kColStep, a0);
                    if (it + 1 < kIters) {
                        tmem_ld_wait();
                        if (it + 2 < kIters) load(col0 + (it + 2) * kColStep, a0);
                        finish(col0 + (it + 1) * kColStep, a1);
                    }
                }
            } else {
                for (int col = part * 8; col < tile_n; col += kColStep) {
                    int acc[R][8];
                    load(col, acc);
                    tmem_ld_wait();
                    finish(col, acc);
                }
            }
        }
    }

    // ------------------------------ teardown ---------------------------------------
    tc_fence_before();
    // PAIR: neither CTA may free tensor memory or leave (its shared memory feeds the
    // partner's MMAs) before both have finished.
    if (PAIR) cluster_sync_all(); else __syncthreads();
    if (threadIdx.x == 0 && ctl.abort) {
        if (p.status != nullptr) atomicExch(p.status, (int)RNS_ERR_DEVICE_TIMEOUT);
        // First CTA to give up records which wait expired and where in the grid.
        if (p.wait_info != nullptr && atomicCAS(p.wait_info, 0, ctl.abort) == 0) {
            p.wait_info[1] = (int)blockIdx.x;
            p.wait_info[2] = (int)blockIdx.y;
            p.wait_info[3] = R * 1000000 + (PAIR ? 100000 : 0) + (FIXED ? 10000 : 0) + tile_n;
        }
    }
    if (warp == 1) {
        tc_fence_after();
        if (PAIR) tmem_dealloc2(tmem_base, (uint32_t)p.tmem_cols);
        else tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
    }
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    });
    return fn;
}

static int make_map(CUtensorMap* map, const void* base, int rank, const uint64_t* dims,
                    const uint64_t* strides_bytes, const uint32_t* box, int tile_k) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return fail(RNS_ERR_CUDA, "cuTensorMapEncodeTiled is unavailable in this driver");
    cuuint64_t gdim[3];
    cuuint64_t gstr[2];
    cuuint32_t bx[3];
    cuuint32_t es[3] = {1, 1, 1};
    for (int i = 0; i < rank; ++i) { gdim[i] = dims[i]; bx[i] = box[i]; }
    for (int i = 0; i + 1 < rank; ++i) gstr[i] = strides_bytes[i];
    const CUresult rc = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, (cuuint32_t)rank,
                           const_cast<void*>(base), gdim, gstr, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           tile_k == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) return fail(RNS_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d)", (int)rc);
    return RNS_OK;
}

constexpr int kSmemBudget = 227 * 1024 - 2048;  // dynamic bytes we allow ourselves

static int round_up_pow2(int v) {
    int r = 32;
    while (r < v) r <<= 1;
    return r;
}

static bool tc_supported(const Plan& pl, int k, int64_t lda, int64_t ldw, bool exact, const char** why) {
    if (pl.channels < 2 || pl.channels > RNS_TC_MAX_CHANNELS) { *why = "channel count outside 2..8"; return false; }
    if (exact && !pl.encode_single_fold) { *why = "exactly centred residues need every modulus >= 86"; return false; }
    if (k <= 0 || k % 16 != 0) { *why = "K must be a positive multiple of 16"; return false; }
    if (lda % 16 != 0 || ldw % 16 != 0) { *why = "row strides must be multiples of 16 bytes"; return false; }
    return true;
}

template <int R, bool PAIR, int J_ = 0, int ES_ = 0, int PS_ = 0, int RS_ = 0, int G_ = 0>
static int launch(const CUtensorMap& ma, const CUtensorMap& mw, const GemmParams& gp, dim3 grid,
                  size_t smem, cudaStream_t st) {
    // The opt-in shared-memory size is a per-device function attribute: set it on
    // the first launch of this instantiation on each device.
    static std::atomic<uint64_t> configured{0};
    int dev = 0;
    RNS_CUDA_OK(cudaGetDevice(&dev));
    const uint64_t bit = 1ull << (dev & 63);
    if (!(configured.load(std::memory_order_acquire) & bit)) {
        RNS_CUDA_OK(cudaFuncSetAttribute(rns_gemm_kernel<R, PAIR, J_, ES_, PS_, RS_, G_>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         227 * 1024 - 1024));
        configured.fetch_or(bit, std::memory_order_release);
    }
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    if (PAIR) {
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    const cudaError_t rc = cudaLaunchKernelEx(&cfg, rns_gemm_kernel<R, PAIR, J_, ES_, PS_, RS_, G_>, ma, mw, gp);
    if (rc != cudaSuccess) {
        int clusters = -1;
        if (PAIR) cudaOccupancyMaxActiveClusters(&clusters, rns_gemm_kernel<R, PAIR, J_, ES_, PS_, RS_, G_>, &cfg);
        cudaGetLastError();
        return fail(RNS_ERR_CUDA, "launch of the RNS GEMM failed: %s (grid %u x %u, smem %zu, pair %d, "
                    "max active clusters %d)", cudaGetErrorString(rc), grid.x, grid.y, smem, (int)PAIR, clusters);
    }
    return RNS_OK;
}

template <int R>
static int launch_either(bool pair, const CUtensorMap& ma, const CUtensorMap& mw, const GemmParams& gp,
                         dim3 grid, size_t smem, cudaStream_t st) {
    return pair ? launch<R, true>(ma, mw, gp, grid, smem, st) : launch<R, false>(ma, mw, gp, grid, smem, st);
}

// rns_gemm_tmem_sm100.cu
bool tmem_gemm_supported(const rns_linear_args* a);
int launch_tmem_gemm(const rns_linear_args* a, const Plan& plan, cudaStream_t st);
// rns_gemm_pair_sm100.cu
int pair_gemm_token_tile(int channels);
bool pair_gemm_supported(const rns_linear_args* a);
int launch_pair_gemm(const rns_linear_args* a, const Plan& plan, cudaStream_t st);

}  // namespace rns

using namespace rns;

extern "C" {

int rns_linear_fused_supported(const int32_t* moduli, int channels, int k, int64_t lda, int64_t ldw) {
    Plan pl;
    if (build_plan(moduli, channels, &pl) != RNS_OK) return 0;
    const char* why = "";
    return tc_supported(pl, k, lda, ldw, false, &why) ? 1 : 0;
}

int rns_pair_tile_rows(int channels, int k) {
    if (channels < 4 || channels > 6 || k < 8 * kPackK || k % 16 != 0) return 0;
    return pair_gemm_token_tile(channels) / 2;
}

int rns_linear_fused(const rns_linear_args* a, rns_stream_t stream) {
    if (!a) return fail(RNS_ERR_INVALID_ARGUMENT, "args is NULL");
    GemmParams gp;
    memset(&gp, 0, sizeof(gp));
    if (int rc = build_plan(a->moduli, a->channels, &gp.plan)) return rc;
    if (a->m <= 0 || a->n <= 0 || a->k <= 0)
        return fail(RNS_ERR_INVALID_ARGUMENT, "matrix dimensions must be positive");
    if ((a->d_a == nullptr) == (a->d_a_planes == nullptr))
        return fail(RNS_ERR_INVALID_ARGUMENT, "give exactly one of d_a and d_a_planes");
    if (!a->d_w || !a->d_out) return fail(RNS_ERR_INVALID_ARGUMENT, "d_w and d_out must be non-NULL");
    const bool planes = a->d_a_planes != nullptr;
    const bool a_packed = a->a_packed != 0, w_packed = a->w_packed != 0;
    if ((!a_packed && a->lda < a->k) || (!w_packed && a->ldw < a->k) || a->ldo < a->n)
        return fail(RNS_ERR_INVALID_ARGUMENT, "a leading dimension is smaller than its row");
    if (planes && !a_packed && a->a_plane_stride < (int64_t)(a->m - 1) * a->lda + a->k)
        return fail(RNS_ERR_INVALID_ARGUMENT, "a_plane_stride is smaller than one plane");
    if (a->out_type < RNS_OUT_INT64 || a->out_type > RNS_OUT_F32)
        return fail(RNS_ERR_INVALID_ARGUMENT, "unknown out_type");
    const bool is_float = a->out_type >= RNS_OUT_F16;
    if (is_float && (!a->d_row_scale || !a->d_col_scale))
        return fail(RNS_ERR_INVALID_ARGUMENT, "floating outputs need d_row_scale and d_col_scale");
    if (is_float && a->row_scale_stride != 0 && a->row_scale_stride != 1)
        return fail(RNS_ERR_INVALID_ARGUMENT, "row_scale_stride must be 0 or 1");
    const Plan& pl = gp.plan;
    const int R = pl.channels;
    if (a->out_type == RNS_OUT_INT32 && (pl.product[R] >> 1) >= (1ll << 31))
        return fail(RNS_ERR_OVERFLOW, "int32 output needs product(moduli)/2 < 2^31");
    const char* why = "";
    if (!tc_supported(pl, a->k, a_packed ? 16 : a->lda, w_packed ? 16 : a->ldw, a->exact_residues != 0, &why))
        return fail(RNS_ERR_UNSUPPORTED, "tensor-core path: %s", why);
    // The per-channel sums are int32: |sum| <= K * 128 * 128 must fit (a wrapped sum is
    // no longer congruent to the true one modulo m).
    if ((int64_t)a->k * 128 * 128 > (int64_t)INT32_MAX)
        return fail(RNS_ERR_OVERFLOW, "K = %d: a channel's int32 sum could exceed 2^31 - 1 (K <= 131071)", a->k);
    if ((a_packed || w_packed) && a->tile_k == 128)
        return fail(RNS_ERR_INVALID_ARGUMENT, "packed operands use tile_k = 64");
    if (planes && !a_packed && a->a_plane_stride % 16 != 0)
        return fail(RNS_ERR_UNSUPPORTED, "tensor-core path: a_plane_stride must be a multiple of 16");
    const void* a_base = planes ? (const void*)a->d_a_planes : (const void*)a->d_a;
    if ((reinterpret_cast<uintptr_t>(a_base) & 15) || (reinterpret_cast<uintptr_t>(a->d_w) & 15))
        return fail(RNS_ERR_UNSUPPORTED, "tensor-core path: operand bases must be 16-byte aligned");

    // ---- kernel variant -----------------------------------------------------
    // 1: both operands staged in shared memory; 2: weights as tensor-memory operands
    // (packed planes + packed weights only).  Variant 2 is limited to 64-token tiles by
    // the 512 tensor-memory columns and measured slower (775 vs 1050 channel-TOPS at
    // 4096^3, four channels), so 0 always resolves to 1; 2 stays selectable.
    if (a->variant < 0 || a->variant > 4) return fail(RNS_ERR_INVALID_ARGUMENT, "variant must be 0, 1, 2, 3 or 4");
    // 3 and 4: the two-CTA feature-major kernels, the only ones that read planes in tiles
    // of a_tile_rows != 128 rows, so that layout selects them (4 unless 3 is asked for).
    // 4 feeds every channel the int8 weight itself, 3 encodes canonical weight residues.
    if (a->variant >= 3 || (a->a_tile_rows != 0 && a->a_tile_rows != kPackM)) {
        if (a->variant != 0 && a->variant < 3)
            return fail(RNS_ERR_INVALID_ARGUMENT, "planes in tiles of %d rows are read by variants 3 and 4 only", a->a_tile_rows);
        if (!pair_gemm_supported(a))
            return fail(RNS_ERR_UNSUPPORTED, "variants 3 and 4 need packed planes in tiles of 64 (4 channels), 48 (5) or 32 "
                                             "(6, variant 4 without output copies) rows, packed weights, all channels active "
                                             "and K >= 512 (grouped calls: K >= 64, whole token tiles, N %% 8 == 0); "
                                             "per-channel weights (w_channel_stride) are read by variant 4 only");
        if (is_float && a->d_absmax_out != nullptr && a->row_scale_stride != 0)
            return fail(RNS_ERR_INVALID_ARGUMENT, "d_absmax_out serves per-tensor scales");
        if (a->n_out_copies < 0 || a->n_out_copies > RNS_MAX_PEERS)
            return fail(RNS_ERR_INVALID_ARGUMENT, "n_out_copies must be in [0, %d]", RNS_MAX_PEERS);
        if (a->n_out_copies > 0 && !is_float)
            return fail(RNS_ERR_INVALID_ARGUMENT, "output copies serve floating outputs");
        for (int g = 0; g < a->n_out_copies; ++g)
            if (!a->d_out_copies[g] || (a->d_absmax_out != nullptr && !a->d_absmax_copies[g]))
                return fail(RNS_ERR_INVALID_ARGUMENT, "d_out_copies / d_absmax_copies hold a NULL pointer");
        return launch_pair_gemm(a, pl, reinterpret_cast<cudaStream_t>(stream));
    }
    if (a->d_absmax_out != nullptr || a->n_out_copies != 0 || a->w_channel_stride != 0 || a->groups != 0)
        return fail(RNS_ERR_UNSUPPORTED, "d_absmax_out, output copies, per-channel weights and grouped calls are served by "
                                         "the two-CTA kernels (tiled planes) only");
    if (a->variant == 2 && !tmem_gemm_supported(a))
        return fail(RNS_ERR_UNSUPPORTED, "variant 2 needs packed planes, packed weights and 2..5 channels");
    if (a->variant == 2)
        return launch_tmem_gemm(a, pl, reinterpret_cast<cudaStream_t>(stream));

    // ---- tile configuration -------------------------------------------------
    const int max_tile_n = ((512 / R) / 16) * 16 > 128 ? 128 : ((512 / R) / 16) * 16;
    int tile_k = a->tile_k;
    if (tile_k == 0) tile_k = 64;
    if (tile_k != 64 && tile_k != 128) return fail(RNS_ERR_INVALID_ARGUMENT, "tile_k must be 64 or 128");
    int tile_n = a->tile_n;
    int m_tiles = (a->m + kTileM - 1) / kTileM;
    // Pair mode (two CTAs per 256 x tile_n tile): 1 = on, 0 = off, anything else = choose.
    // It pays when there are enough tiles to fill the GPU twice over and the W half
    // tile stays at 64 rows (up to four channels; with five the tile is 96 wide and
    // single-CTA tiles measured faster).
    bool pair = a->pair_mode == 1;
    if (a->pair_mode != 0 && a->pair_mode != 1) {
        pair = R <= 4 && m_tiles >= 2 && (int64_t)m_tiles * ((a->n + 127) / 128) >= 2 * 148;
        // With the compile-time ring configuration (see the dispatch below) single-CTA
        // tiles measured faster than pairs (1.69 against 1.54 channel-POPS at 4096^3).
        if (R == 4 && planes && a_packed && w_packed && a->d_active_channels == nullptr &&
            a->exact_residues == 0 && a->k >= 4 * 64)
            pair = false;
    }
    if (pair && tile_k == 128) return fail(RNS_ERR_INVALID_ARGUMENT, "pair mode uses tile_k = 64");
    const int kblocks_hint = (a->k + tile_k - 1) / tile_k;
    if (tile_n == 0) {
        // Largest tile that still gives every SM a CTA; small problems take the
        // narrowest tile so that more SMs stream the weights.
        tile_n = 32;
        const int cands[] = {128, 96, 64, 48, 32};
        for (int c : cands) {
            if (c > max_tile_n) continue;
            if ((int64_t)m_tiles * ((a->n + c - 1) / c) >= 148) { tile_n = c; break; }
        }
        if (tile_n > max_tile_n) tile_n = max_tile_n;
        // Many-token calls on packed planes always take the full-width tile, i.e. the
        // instantiations with compile-time ring parameters, even when that leaves a few
        // SMs without a CTA: a narrower tile would select the run-time form, and that
        // form launched back to back between the fixed ones (the rank-local sequence of an
        // 8-way sharded stack) ended with "unspecified launch failure" on some launches.
        if (planes && a_packed && w_packed && (R == 4 || R == 5) && m_tiles >= 4 && !pair &&
            a->d_active_channels == nullptr && a->exact_residues == 0 && kblocks_hint >= 8)
            tile_n = max_tile_n;
        if (pair && tile_n % 32 != 0) tile_n = tile_n + 16 <= max_tile_n ? tile_n + 16 : tile_n - 16;
    }
    if (tile_n < 16 || tile_n > 128 || tile_n % 16 != 0 || tile_n > max_tile_n)
        return fail(RNS_ERR_INVALID_ARGUMENT, "tile_n must be a multiple of 16 in [16, %d]", max_tile_n);
    if (w_packed && kPackNPad % tile_n != 0)
        return fail(RNS_ERR_INVALID_ARGUMENT, "packed weights need a tile_n that divides %d", kPackNPad);

    if (pair && tile_n % 32 != 0)
        return fail(RNS_ERR_INVALID_ARGUMENT, "pair mode needs tile_n to be a multiple of 32");
    if (pair) m_tiles = (m_tiles + 1) / 2 * 2;
    gp.tile_a_bytes = kTileM * tile_k;
    gp.tile_w_bytes = (pair ? tile_n / 2 : tile_n) * tile_k;
    // Two rings in shared memory.  Raw ring: source bytes as loaded (W tile, and the
    // A tile when activations are not planes).  Operand ring: R tiles for A and for W.
    gp.off_raw_w = 0;
    gp.off_raw_a = gp.tile_w_bytes;
    gp.raw_sub_bytes = (gp.tile_w_bytes + (planes ? 0u : gp.tile_a_bytes) + 1023u) & ~1023u;
    // Operand ring: what the encoders write (W tiles; A tiles too unless activations
    // arrive as planes).  Plane ring: activation planes, operands as loaded.
    gp.off_enc_a = 0;
    gp.off_enc_w = planes ? 0u : R * gp.tile_a_bytes;
    gp.enc_sub_bytes = (R * ((planes ? 0u : gp.tile_a_bytes) + gp.tile_w_bytes) + 1023u) & ~1023u;
    gp.pl_sub_bytes = planes ? R * gp.tile_a_bytes : 0u;
    const int kblocks = (a->k + tile_k - 1) / tile_k;
    if (a->enc_stages < 0 || a->enc_stages > kMaxStages)
        return fail(RNS_ERR_INVALID_ARGUMENT, "enc_stages must be in [0, %d]", kMaxStages);
    if (a->sub_blocks < 0 || a->sub_blocks > 4)
        return fail(RNS_ERR_INVALID_ARGUMENT, "sub_blocks must be in [0, 4]");
    // K blocks per stage (one hand-over per stage; measured: two K blocks per stage and
    // two stages beat four stages of one); never more than leave two stages of every ring.
    const int64_t per_kb = (int64_t)gp.enc_sub_bytes + gp.raw_sub_bytes + gp.pl_sub_bytes;
    int sub_blocks = a->sub_blocks > 0 ? a->sub_blocks : 2;
    while (sub_blocks > 1 && 2 * sub_blocks * per_kb > kSmemBudget) --sub_blocks;
    if (sub_blocks > kblocks) sub_blocks = kblocks;
    gp.sub_blocks = sub_blocks;
    gp.raw_stage_bytes = (uint32_t)sub_blocks * gp.raw_sub_bytes;
    gp.enc_stage_bytes = (uint32_t)sub_blocks * gp.enc_sub_bytes;
    gp.pl_stage_bytes = (uint32_t)sub_blocks * gp.pl_sub_bytes;
    const int nstages = (kblocks + sub_blocks - 1) / sub_blocks;
    // Depths: the operand ring as asked (default 4), the plane ring as deep as the
    // operand ring, and a raw ring at least as deep as the operand ring (the encoders'
    // parity argument needs that); whatever memory is left deepens first the plane
    // ring, then the raw ring (both only hide load latency).
    int enc_stages = a->enc_stages > 0 ? a->enc_stages : 4;
    if (enc_stages > nstages) enc_stages = nstages;
    auto ring_bytes = [&](int e, int pl, int rw) {
        return (int64_t)e * gp.enc_stage_bytes + (int64_t)pl * gp.pl_stage_bytes + (int64_t)rw * gp.raw_stage_bytes;
    };
    while (enc_stages > 1 && ring_bytes(enc_stages, planes ? enc_stages : 0, enc_stages) > kSmemBudget) --enc_stages;
    if (ring_bytes(enc_stages, planes ? enc_stages : 0, enc_stages) > kSmemBudget)
        return fail(RNS_ERR_UNSUPPORTED, "tile configuration does not fit shared memory");
    int pl_stages = planes ? enc_stages : 0, raw_stages = enc_stages;
    const int pl_cap = nstages < kMaxStages ? nstages : kMaxStages;
    while (planes && pl_stages < pl_cap && pl_stages < 6 && ring_bytes(enc_stages, pl_stages + 1, raw_stages) <= kSmemBudget)
        ++pl_stages;
    while (raw_stages < pl_cap && ring_bytes(enc_stages, pl_stages, raw_stages + 1) <= kSmemBudget) ++raw_stages;
    // Single-CTA tiles of the hot configuration read W straight from global memory in
    // the encoder threads: no raw ring, and its memory deepens the operand ring.
    const bool w_direct = !pair && planes && a_packed && w_packed && tile_k == 64 && a->d_active_channels == nullptr &&
                          a->exact_residues == 0 && (R == 4 || R == 5) && tile_n == (R <= 4 ? 128 : 96) &&
                          a->sub_blocks == 0 && a->enc_stages == 0 && a->enc_groups == 0 && kblocks >= 8;
    if (w_direct) {
        sub_blocks = 1;
        gp.sub_blocks = 1;
        gp.raw_stage_bytes = gp.raw_sub_bytes;
        gp.enc_stage_bytes = gp.enc_sub_bytes;
        gp.pl_stage_bytes = gp.pl_sub_bytes;
        raw_stages = 0;
        enc_stages = R == 4 ? 4 : 3;
        pl_stages = 3;
    }
    // ... and with packed int8 activations instead of planes the activation tile too.
    const bool a_direct = !pair && !planes && a_packed && w_packed && tile_k == 64 && a->d_active_channels == nullptr &&
                          a->exact_residues == 0 && (R == 4 || R == 5) && tile_n == (R <= 4 ? 128 : 96) &&
                          a->sub_blocks == 0 && a->enc_stages == 0 && a->enc_groups == 0 && kblocks >= 8;
    if (a_direct) {
        sub_blocks = 1;
        gp.sub_blocks = 1;
        gp.raw_stage_bytes = gp.raw_sub_bytes;
        gp.enc_stage_bytes = gp.enc_sub_bytes;
        gp.pl_stage_bytes = 0;
        raw_stages = 0;
        enc_stages = 3;
        pl_stages = 0;
    }
    gp.raw_stages = raw_stages;
    gp.enc_stages = enc_stages;
    gp.pl_stages = pl_stages > 0 ? pl_stages : 1;
    gp.enc_ring_offset = (uint32_t)raw_stages * gp.raw_stage_bytes;
    gp.pl_ring_offset = gp.enc_ring_offset + (uint32_t)enc_stages * gp.enc_stage_bytes;
    gp.enc_groups = a->enc_groups > 0 ? a->enc_groups : (enc_stages >= 2 ? 2 : 1);
    if (gp.enc_groups != 1 && gp.enc_groups != 2 && gp.enc_groups != 4)
        return fail(RNS_ERR_INVALID_ARGUMENT, "enc_groups must be 1, 2 or 4");
    // A group runs at most one operand slot per member ahead: never more groups than slots.
    while (gp.enc_groups > enc_stages) gp.enc_groups /= 2;
    gp.m = a->m; gp.n = a->n; gp.k = a->k;
    gp.tile_n = tile_n; gp.tile_k = tile_k;
    gp.exact_residues = a->exact_residues ? 1 : 0;
    gp.a_is_planes = planes ? 1 : 0;
    gp.a_packed = a_packed ? 1 : 0;
    gp.w_packed = w_packed ? 1 : 0;
    gp.a_ptr = planes ? a->d_a_planes : a->d_a;
    gp.w_ptr = a->d_w;
    gp.w_npad = round_up_i64(a->n, kPackNPad);
    gp.tmem_cols = round_up_pow2(R * tile_n);
    gp.active_ptr = a->d_active_channels;
    gp.out = a->d_out; gp.ldo = a->ldo; gp.out_type = a->out_type;
    gp.row_scale = a->d_row_scale; gp.row_scale_stride = a->row_scale_stride;
    gp.col_scale = a->d_col_scale; gp.bias = a->d_bias; gp.status = a->d_status;
    gp.wait_info = a->d_wait_info;

    // ---- tensor maps -------------------------------------------------------
    CUtensorMap map_a, map_w;
    memset(&map_a, 0, sizeof(map_a));
    memset(&map_w, 0, sizeof(map_w));
    if (!w_packed) {
        const uint64_t dims[2] = {(uint64_t)a->k, (uint64_t)a->n};
        const uint64_t strides[1] = {(uint64_t)a->ldw};
        const uint32_t box[2] = {(uint32_t)tile_k, (uint32_t)(pair ? tile_n / 2 : tile_n)};
        if (int rc = make_map(&map_w, a->d_w, 2, dims, strides, box, tile_k)) return rc;
    }
    if (a_packed) {
        // bulk copies: no tensor map
    } else if (planes) {
        const uint64_t dims[3] = {(uint64_t)a->k, (uint64_t)a->m, (uint64_t)R};
        const uint64_t strides[2] = {(uint64_t)a->lda, (uint64_t)a->a_plane_stride};
        const uint32_t box[3] = {(uint32_t)tile_k, (uint32_t)kTileM, 1u};
        if (int rc = make_map(&map_a, a_base, 3, dims, strides, box, tile_k)) return rc;
    } else {
        const uint64_t dims[2] = {(uint64_t)a->k, (uint64_t)a->m};
        const uint64_t strides[1] = {(uint64_t)a->lda};
        const uint32_t box[2] = {(uint32_t)tile_k, (uint32_t)kTileM};
        if (int rc = make_map(&map_a, a_base, 2, dims, strides, box, tile_k)) return rc;
    }

    const int n_tiles = (a->n + tile_n - 1) / tile_n;
    const dim3 grid = pair ? dim3(2 * n_tiles, m_tiles / 2, 1) : dim3(n_tiles, m_tiles, 1);
    const size_t smem = (size_t)ring_bytes(enc_stages, pl_stages, raw_stages) + 1024;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    // The hot configurations have instantiations with compile-time ring parameters.
    const bool fixed_ok = planes && a_packed && w_packed && tile_k == 64 && a->d_active_channels == nullptr &&
                          a->exact_residues == 0 && tile_n == (R <= 4 ? 128 : 96);
    auto rings_are = [&](int j, int es, int ps, int rs, int g) {
        return fixed_ok && sub_blocks == j && enc_stages == es && pl_stages == ps && raw_stages == rs &&
               gp.enc_groups == g;
    };
#define RNS_FIXED(r, pr, j, es, ps, rs, g) \
    if (R == r && pair == pr && rings_are(j, es, ps, rs, g)) \
        return launch<r, pr, j, es, ps, rs, g>(map_a, map_w, gp, grid, smem, st);
    // (one encoder group measured best with direct weight loads: 1.80 against 1.72
    // channel-POPS at 4096^3)
    if (a_direct) gp.enc_groups = 1;
    if (a_direct && R == 4) return launch<4, false, 1, 3, 0, -1, 1>(map_a, map_w, gp, grid, smem, st);
    if (a_direct && R == 5) return launch<5, false, 1, 3, 0, -1, 1>(map_a, map_w, gp, grid, smem, st);
    if (w_direct) gp.enc_groups = 1;
    if (w_direct && R == 4) return launch<4, false, 1, 4, 3, -1, 1>(map_a, map_w, gp, grid, smem, st);
    if (w_direct && R == 5) return launch<5, false, 1, 3, 3, -1, 1>(map_a, map_w, gp, grid, smem, st);
    RNS_FIXED(4, false, 1, 3, 3, 4, 2)
    RNS_FIXED(5, false, 1, 2, 3, 7, 2)
    RNS_FIXED(4, true, 2, 2, 2, 4, 2)
#ifdef RNS_MORE_FIXED
    RNS_FIXED(4, false, 1, 3, 3, 4, 1)
    RNS_FIXED(4, false, 1, 2, 4, 4, 2)
    RNS_FIXED(4, false, 1, 2, 4, 4, 1)
    RNS_FIXED(5, false, 1, 2, 3, 7, 1)
    RNS_FIXED(4, true, 2, 2, 2, 4, 1)
    RNS_FIXED(4, true, 1, 4, 4, 8, 2)
    RNS_FIXED(4, true, 1, 4, 4, 8, 4)
    RNS_FIXED(4, true, 1, 3, 5, 4, 2)
    RNS_FIXED(4, true, 1, 2, 6, 4, 2)
#endif
#undef RNS_FIXED
    switch (R) {
        case 2: return launch_either<2>(pair, map_a, map_w, gp, grid, smem, st);
        case 3: return launch_either<3>(pair, map_a, map_w, gp, grid, smem, st);
        case 4: return launch_either<4>(pair, map_a, map_w, gp, grid, smem, st);
        case 5: return launch_either<5>(pair, map_a, map_w, gp, grid, smem, st);
        case 6: return launch_either<6>(pair, map_a, map_w, gp, grid, smem, st);
        case 7: return launch_either<7>(pair, map_a, map_w, gp, grid, smem, st);
        case 8: return launch_either<8>(pair, map_a, map_w, gp, grid, smem, st);
        default: return fail(RNS_ERR_UNSUPPORTED, "tensor-core path: channel count outside 2..8");
    }
}

}  // extern "C"
