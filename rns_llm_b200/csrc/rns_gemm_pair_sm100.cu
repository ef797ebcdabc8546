// Fused RNS linear for many-token calls on sm_100a: two CTAs of a cluster compute one
// 256-feature x TOK-token output tile with tcgen05 cta_group::2.
//
// Roles of the operands are swapped against rns_gemm_sm100.cu.  The weight rows are the
// MMA's M operand: each CTA owns 128 output features, reads its 128 x 64 bytes of the
// packed weight per K block straight from global memory and encodes them into R residue
// tiles in shared memory.  The tokens are the N operand, which cta_group::2 splits over
// the pair: each CTA bulk-copies only HALF of the token tile's residue planes
// (R x TOK/2 x 64 bytes per K block), so the L2 -> SM traffic per CTA and K block drops
// from R x 8 KB + 8 KB to R x 4 KB + 8 KB, and a deeper plane ring fits shared memory.
// Accumulators: R x TOK int32 columns of tensor memory in each CTA (its 128 features as
// lanes); the epilogue is feature-major (a thread owns one feature, walks the tokens).
//
// Per CTA: warp 0 loads planes; warp 1 issues the MMAs (leader CTA) or tells the leader
// that this CTA's stage is complete (peer CTA); warps 2..17 encode weights during the K
// loop and run the epilogue.  One tcgen05.commit per stage, multicast to both CTAs,
// releases the operand slot and the plane slot of that stage through one ring of
// "stage done" barriers.  Every wait is bounded (status word + wait code on expiry).
#include "rns_pair.cuh"

namespace rns {


// Persistent: a cluster walks the tiles cluster, cluster + clusters, ...  All rings run on
// one stage counter g that keeps counting across tiles (slot = g mod depth), so the loads
// and the weight encoding of the next tile start while this tile's last MMAs and its
// epilogue are still running; only the MMAs wait for the accumulators to be drained.
// COPIES: the instantiation that also stores into the other ranks' buffers; the plain one
// carries none of that code.
template <int R, int TOK, int ES, int PS, bool COPIES>
__global__ void __launch_bounds__(kPairThreads, 1)
rns_gemm_pair_kernel(const __grid_constant__ PairParams p) {
    static_assert(R * TOK <= 512, "accumulators must fit tensor memory");
    static_assert(TOK % 16 == 0 && (TOK / 2) % 8 == 0, "token tile shape");
    static_assert(ES <= kDoneRing && PS <= kDoneRing && ES >= kPairGroups, "ring depths");
    // An issuer warp takes every other stage.  With even ring depths a slot is always
    // handled by the same warp, which therefore sees every phase of the slot's barrier; with
    // an odd depth it would skip alternate phases and could mistake "the phase before last
    // has completed" for the one it waits for (a parity wait cannot tell them apart).
    static_assert(ES % 2 == 0 && PS % 2 == 0 && kDoneRing % 2 == 0, "ring depths must be even");
    constexpr int TR = TOK / 2;                               // token rows this CTA loads
    constexpr uint32_t kOpStage = (uint32_t)R * kPairOpTile;
    constexpr uint32_t kPlTile = (uint32_t)TR * kPackK;
    constexpr uint32_t kPlStage = (uint32_t)R * kPlTile;
    constexpr uint32_t kTmemCols = 512;

    extern __shared__ uint8_t smem_dyn[];
    __shared__ PairCtl ctl;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t tiles_base = (smem_addr(smem_dyn) + 1023u) & ~1023u;
    uint8_t* tiles_ptr = smem_dyn + (tiles_base - smem_addr(smem_dyn));
    const uint32_t op_base = tiles_base;                       // operand ring first
    const uint32_t pl_base = tiles_base + (uint32_t)ES * kOpStage;

    const uint32_t rank = cluster_cta_rank();
    const int cluster = (int)(blockIdx.x >> 1), clusters = (int)(gridDim.x >> 1);
    const int tiles = p.n_ftiles * p.n_ttiles;
    const int nst = p.kblocks;                                 // one K block of 64 bytes per stage

    if (threadIdx.x == 0) {
        ctl.abort = 0;
        ctl.absmax = 0u;
        for (int s = 0; s < kDoneRing; ++s) {
            // The leader's barriers collect the peer CTA's arrivals too: its encoder warps
            // arrive on the leader's full_op directly, its plane load through a relay lane.
            mbar_init(smem_addr(&ctl.full_op[s]), 2 * kPairGroupWarps);
            mbar_init(smem_addr(&ctl.full_pl[s]), rank == 0 ? 2 : 1);
            mbar_init(smem_addr(&ctl.done[s]), 1);
        }
        mbar_init(smem_addr(&ctl.acc_full), 2);                // one commit from each issuer warp
        mbar_init(smem_addr(&ctl.tmem_free), 2 * kPairEncWarps);   // leader: both CTAs' epilogue warps
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc2(smem_addr(&ctl.tmem_base), kTmemCols);
        tmem_relinquish2();
    }
    tc_fence_before();
    cluster_sync_all();                 // both CTAs' barriers exist before either signals the other
    tc_fence_after();
    const uint32_t tmem_base = ctl.tmem_base;
    volatile int* abort = &ctl.abort;

    if (warp == kPairPlaneWarp) {
        // ------------------------------ plane producer ----------------------------
        if (lane == 0) {
            int g = 0;
            bool ok = true;
            for (int tile = cluster; tile < tiles && ok; tile += clusters) {
                const PairTile t = pair_tile<TOK>(p, tile, rank);
                const int8_t* src = p.planes + ((int64_t)(t.tt * 2 + (int)rank) * p.kblocks) * (int64_t)kPlStage;
                for (int st = 0; st < nst; ++st, ++g) {
                    if (g >= PS &&
                        !wait_bounded<false, true>(smem_addr(&ctl.done[(g - PS) & (kDoneRing - 1)]),
                                                   (uint32_t)((g - PS) >> 3) & 1u, abort, wait_code(2, st))) {
                        ok = false;
                        break;
                    }
                    const int sp = g % PS;
                    const uint32_t bar = smem_addr(&ctl.full_pl[sp]);
                    mbar_arrive_expect_tx(bar, kPlStage);
                    bulk_load(pl_base + (uint32_t)sp * kPlStage, src + (int64_t)st * kPlStage, kPlStage, bar);
                }
            }
        }
        __syncwarp();
    } else if (warp <= 1) {
        const int my_tiles = (tiles - cluster + clusters - 1) / clusters;
        const int total = my_tiles * nst;                      // stages this cluster runs
        if (rank != 0) {
            // ------------------------------ plane relay (peer CTA) ----------------
            // Tells the leader that this CTA's plane half of a stage has landed.  Planes
            // run several stages ahead of the MMAs, so this hop is off the critical path.
            if (warp == 1 && lane == 0) {
                for (int g = 0; g < total; ++g) {
                    if (!wait_bounded<false, true>(smem_addr(&ctl.full_pl[g % PS]), (uint32_t)(g / PS) & 1u, abort,
                                                   wait_code(4, g))) break;
                    mbar_arrive_remote_relaxed(smem_addr(&ctl.full_pl[g % PS]), 0);
                }
            }
            __syncwarp();
        } else {
            // ------------------------------ MMA issuers (leader CTA) ---------------
            // Two warps take alternate stages: an issuer's instruction stream per stage
            // (two barrier tests, eight MMAs, a commit) is longer than the MMAs run, so
            // one of them cannot keep the tensor pipe fed.  Integer accumulation does not
            // depend on the order of the MMAs; the epilogue warps leave the accumulators
            // zeroed, so that no MMA has to come first.  Each whole warp runs the loop
            // (addresses and descriptors are then warp-uniform values); one elected lane
            // issues.
            const uint32_t idesc = make_idesc(256u, (uint32_t)TOK);
            const uint64_t desc0 = make_smem_desc(0, kPackK);
            const uint32_t a_lo0 = op_base >> 4, b_lo0 = pl_base >> 4;
            bool ok = true;
            int g0 = 0;                                        // first stage of the current tile
            for (int ti = 0; ti < my_tiles && ok; ++ti, g0 += nst) {
                // accumulators drained and zeroed (by both CTAs) since the previous tile
                ok = warp_wait_bounded<false, true>(smem_addr(&ctl.tmem_free), (uint32_t)ti & 1u, abort, wait_code(9, ti));
                if (!ok) break;
                for (int g = g0 + ((g0 + warp) & 1); g < g0 + nst; g += 2) {
                    const int s = g % ES, sp = g % PS;
                    ok = warp_wait_bounded<false, true>(smem_addr(&ctl.full_op[s]), (uint32_t)(g / ES) & 1u, abort, wait_code(5, g));
                    if (ok) ok = warp_wait_bounded<false, true>(smem_addr(&ctl.full_pl[sp]), (uint32_t)(g / PS) & 1u, abort, wait_code(6, g));
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t a_st = a_lo0 + (uint32_t)s * (kOpStage >> 4);
                    const uint32_t b_st = b_lo0 + (uint32_t)sp * (kPlStage >> 4);
                    if (elect_one()) {
#pragma unroll
                        for (int c = 0; c < R; ++c) {
#pragma unroll
                            for (int ks = 0; ks < 2; ++ks) {
                                const uint64_t da = desc0 | (uint64_t)(a_st + (uint32_t)c * (kPairOpTile >> 4) + (uint32_t)ks * 2u);
                                const uint64_t db = desc0 | (uint64_t)(b_st + (uint32_t)c * (kPlTile >> 4) + (uint32_t)ks * 2u);
                                umma_i8_pair(tmem_base + (uint32_t)(c * TOK), da, db, idesc, 1u);
                            }
                        }
                        umma_commit_pair(smem_addr(&ctl.done[g & (kDoneRing - 1)]));
                    }
                    __syncwarp();
                }
                // this warp's MMAs of the tile are in the pipe: the accumulators are complete
                // when both warps' commits have arrived
                if (ok && elect_one()) umma_commit_pair(smem_addr(&ctl.acc_full));
                __syncwarp();
            }
        }
    } else {
        // ------------------------------ encoders / epilogue ------------------------
        const int quarter = warp & 3;                          // tensor-memory lanes 32*quarter .. +31
        const int part = (warp - 2) >> 2;                      // quarter of the token columns
        const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
        // Zeroes this warp's share of the accumulators (its lane quarter, 128 of the 512
        // columns) and tells the leader's issuers.
        auto zero_and_release = [&]() {
            uint32_t zeros[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) zeros[i] = 0u;
#pragma unroll
            for (int i = 0; i < 8; ++i) tmem_st16(lane_base + (uint32_t)(part * 128 + i * 16), zeros);
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (rank == 0) mbar_arrive(smem_addr(&ctl.tmem_free));
                else mbar_arrive_remote_relaxed(smem_addr(&ctl.tmem_free), 0);
            }
        };
        zero_and_release();
        const int group = (warp - 2) & (kPairGroups - 1);
        const int e0 = ((warp - 2) / kPairGroups) * 32 + lane;  // first 16-byte chunk of this thread
        uint32_t mfold[R];
#pragma unroll
        for (int c = 0; c < R; ++c) mfold[c] = p.plan.enc_mfold[c];
        const int64_t kb_stride = p.w_npad * kPackK;
        const bool is_float = p.out_type >= RNS_OUT_F16;
        const float rs_all = (is_float && p.row_scale_stride == 0) ? p.row_scale[0] : 0.0f;
        float biggest = 0.0f;
        bool ok = true;
        int g0 = 0, ti = 0;
        for (int tile = cluster; tile < tiles && ok; tile += clusters, ++ti, g0 += nst) {
            const PairTile t = pair_tile<TOK>(p, tile, rank);
            const int n0 = t.n0, tok0 = t.tok0;
            // -------- weight encoding: this group's stages of the tile --------
            const int8_t* w_src = p.w + (int64_t)n0 * kPackK + (int64_t)e0 * 16;
            bool valid[kPairChunks];
#pragma unroll
            for (int i = 0; i < kPairChunks; ++i) valid[i] = n0 + ((e0 + i * kPairGroupThreads) >> 2) < p.n;
            auto load_w = [&](int st, uint4 (&dst)[kPairChunks]) {
#pragma unroll
                for (int i = 0; i < kPairChunks; ++i) {
                    if (valid[i] && st < nst)
                        dst[i] = __ldg(reinterpret_cast<const uint4*>(w_src + (int64_t)st * kb_stride + (int64_t)i * kPairGroupThreads * 16));
                    else
                        dst[i] = make_uint4(0u, 0u, 0u, 0u);
                }
            };
            const int st_first = (g0 + group) & 1;             // stages with g = group (mod 2)
            uint4 cur[kPairChunks], nxt[kPairChunks];
            load_w(st_first, cur);
            load_w(st_first + kPairGroups, nxt);
            for (int st = st_first; st < nst && ok; st += kPairGroups) {
                const int g = g0 + st;
                const int s = g % ES;
                uint4 ahead[kPairChunks];
                load_w(st + 2 * kPairGroups, ahead);
                if (g >= ES)
                    ok = warp_wait_bounded(smem_addr(&ctl.done[(g - ES) & (kDoneRing - 1)]),
                                           (uint32_t)((g - ES) >> 3) & 1u, abort, wait_code(8, g));
                if (!ok) break;
                uint8_t* dst = tiles_ptr + (size_t)s * kOpStage + (size_t)e0 * 16;
#pragma unroll
                for (int i = 0; i < kPairChunks; ++i) {
                    const uint4 x = cur[i];
                    const uint32_t u0 = x.x ^ 0x80808080u, u1 = x.y ^ 0x80808080u;
                    const uint32_t u2 = x.z ^ 0x80808080u, u3 = x.w ^ 0x80808080u;
                    const uint32_t d0 = fold_pattern(x.x), d1 = fold_pattern(x.y);
                    const uint32_t d2 = fold_pattern(x.z), d3 = fold_pattern(x.w);
#pragma unroll
                    for (int c = 0; c < R; ++c) {
                        uint4 y;
                        y.x = encode_word_reduced(u0, d0, mfold[c]);
                        y.y = encode_word_reduced(u1, d1, mfold[c]);
                        y.z = encode_word_reduced(u2, d2, mfold[c]);
                        y.w = encode_word_reduced(u3, d3, mfold[c]);
                        *reinterpret_cast<uint4*>(dst + (size_t)i * kPairGroupThreads * 16 + (size_t)c * kPairOpTile) = y;
                    }
                }
#pragma unroll
                for (int i = 0; i < kPairChunks; ++i) { cur[i] = nxt[i]; nxt[i] = ahead[i]; }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    if (rank == 0) mbar_arrive(smem_addr(&ctl.full_op[s]));
                    else mbar_arrive_remote_relaxed(smem_addr(&ctl.full_op[s]), 0);
                }
            }

            // -------- epilogue of the tile (feature-major) --------
            if (ok) ok = warp_wait_bounded(smem_addr(&ctl.acc_full), (uint32_t)ti & 1u, abort, wait_code(11, ti));
            if (!ok) break;
            tc_fence_after();
            pair_epilogue<R, TOK, COPIES, false, false>(p, n0, tok0, quarter, part, lane, lane_base, is_float, rs_all, biggest, [] {});
            // Every column this warp read belongs to channel blocks c*TOK + [col0, col0 + TOK/4);
            // the columns it ZEROES are its 128-column block.  All sixteen warps have to be
            // done reading before anyone's zeroes may land on columns another warp still reads.
            asm volatile("bar.sync 1, %0;" ::"n"(kPairEncWarps * 32) : "memory");
            zero_and_release();
        }
        if (p.absmax_out != nullptr && is_float) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) biggest = fmaxf(biggest, __shfl_xor_sync(0xffffffffu, biggest, o));
            if (lane == 0) atomicMax(&ctl.absmax, __float_as_uint(biggest));
        }
    }

    // ------------------------------ teardown ---------------------------------------
    // Nothing may still be on its way to this CTA's barriers when it leaves: the last
    // stages' commits are waited for here (nobody else waits for them).
    if (warp == 1 && lane == 0 && !*abort) {
        const int total = ((tiles - cluster + clusters - 1) / clusters) * nst;
        for (int g = total > kDoneRing ? total - kDoneRing : 0; g < total; ++g)
            if (!wait_bounded(smem_addr(&ctl.done[g & (kDoneRing - 1)]), (uint32_t)(g >> 3) & 1u, abort,
                              wait_code(12, g)))
                break;
    }
    tc_fence_before();
    // Neither CTA may free tensor memory or leave (its shared memory feeds the partner's
    // MMAs, its barriers receive the partner's arrivals) before both have finished.
    cluster_sync_all();
    if (threadIdx.x == 0) {
        if (ctl.abort) {
            if (p.status != nullptr) atomicExch(p.status, (int)RNS_ERR_DEVICE_TIMEOUT);
            if (p.wait_info != nullptr && atomicCAS(p.wait_info, 0, ctl.abort) == 0) {
                p.wait_info[1] = (int)blockIdx.x;
                p.wait_info[2] = (int)blockIdx.y;
                p.wait_info[3] = R * 1000000 + 200000 + TOK;
            }
        } else if (p.absmax_out != nullptr) {
            if (ctl.absmax != 0u) atomicMax(p.absmax_out, ctl.absmax);
            if (COPIES && p.n_copies > 0) {
                // The last CTA to contribute hands the finished word to the other ranks.
                __threadfence();
                if (atomicAdd(p.absmax_out + 1, 1u) == gridDim.x - 1) {
                    const uint32_t final_word = atomicMax(p.absmax_out, 0u);
                    for (int g = 0; COPIES && g < p.n_copies; ++g) *p.absmax_copies[g] = final_word;
                }
            }
        }
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc2(tmem_base, kTmemCols);
    }
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
template <int R, int TOK, int ES, int PS, bool COPIES>
static int launch_pair(const PairParams& pp, int pairs, cudaStream_t st) {
    constexpr size_t smem = (size_t)ES * R * kPairOpTile + (size_t)PS * R * (TOK / 2) * kPackK + 1024;
    static_assert(smem + sizeof(PairCtl) <= 227 * 1024, "rings exceed shared memory");
    return launch_pair_clusters<rns_gemm_pair_kernel<R, TOK, ES, PS, COPIES>>(smem, pp, pairs, st);
}

int pair_gemm_token_tile(int channels) { return pair_raw_token_tile(channels); }

// Grouped calls: the plain raw-weight form only, whole token tiles, weight rows in eights.
static bool pair_groups_ok(const rns_linear_args* a) {
    if (a->groups <= 0) return a->groups == 0;
    return a->variant != 3 && a->w_channel_stride == 0 && a->n_out_copies == 0 && a->d_active_channels == nullptr &&
           a->d_absmax_out == nullptr && a->m % pair_gemm_token_tile(a->channels) == 0 && a->n % 8 == 0 &&
           (int64_t)a->groups * a->m <= INT32_MAX && (int64_t)a->groups * a->n <= INT32_MAX;
}

// 4, 5 or 6 channels (the weight-encoding kernel, variant 3, and output copies: 4 or 5).
bool pair_gemm_supported(const rns_linear_args* a) {
    const bool channels_ok = a->channels == 4 || a->channels == 5 ||
                             (a->channels == 6 && a->variant != 3 && a->n_out_copies == 0);
    // an adaptive prefix (d_active_channels) is honoured by the raw-weight kernel with one weight matrix
    const bool prefix_ok = a->d_active_channels == nullptr ||
                           (a->variant != 3 && a->w_channel_stride == 0 && a->n_out_copies == 0 && a->channels <= 5);
    return a->d_a_planes != nullptr && a->a_packed != 0 && a->w_packed != 0 && prefix_ok &&
           a->exact_residues == 0 && channels_ok && (a->w_channel_stride == 0 || a->variant != 3) &&
           a->w_channel_stride >= 0 && a->w_channel_stride % 16 == 0 &&
           a->a_tile_rows == pair_gemm_token_tile(a->channels) / 2 && a->k % 16 == 0 &&
           a->k >= (a->groups >= 1 ? kPackK : 8 * kPackK) && pair_groups_ok(a);
}

int launch_pair_gemm(const rns_linear_args* a, const Plan& plan, cudaStream_t st) {
    PairParams pp;
    memset(&pp, 0, sizeof(pp));
    pp.plan = plan;
    const int R = plan.channels;
    const int tok = pair_gemm_token_tile(R);
    pp.m = a->m; pp.n = a->n; pp.k = a->k;
    pp.kblocks = (a->k + kPackK - 1) / kPackK;
    pp.planes = a->d_a_planes;
    pp.w = a->d_w;
    const int groups = a->groups > 1 ? a->groups : 1;
    pp.w_npad = round_up_i64((int64_t)groups * a->n, kPackNPad);
    pp.w_channel_stride = a->w_channel_stride;
    pp.groups = groups;
    pp.w_group_rows = a->n;
    pp.out_group_stride = (int64_t)a->m * a->ldo;
    pp.n_ftiles = (a->n + 255) / 256;
    pp.n_ttiles = (a->m + tok - 1) / tok;
    // Band: as many feature tiles as keep the band's weight bytes around 32 MB (a quarter
    // of L2), at least the number that fills the GPU once with one token tile each.
    // (Per-channel weight planes count R times: with one byte per value assumed, the bands of
    // a five-channel wide layer held 160 MB and the launch read 4.5 GB from DRAM, 13 times
    // its operands.)
    // Measured on the wide QKV / fc2 shapes: 32 MB suits K = 4096, 96 MB K = 16384, where every
    // band re-reads 335 MB of planes.
    const int64_t band_bytes = (a->w_channel_stride != 0 && a->k >= 8192 ? 96ll : 32ll) << 20;
    const int64_t weight_copies = a->w_channel_stride != 0 ? R : 1;
    int band = (int)(band_bytes / ((int64_t)256 * pp.kblocks * kPackK * weight_copies));
    if (band < 1) band = 1;
    if (band > pp.n_ftiles) band = pp.n_ftiles;
    pp.band = band;
    pp.out = a->d_out; pp.ldo = a->ldo; pp.out_type = a->out_type;
    pp.row_scale = a->d_row_scale; pp.row_scale_stride = a->row_scale_stride;
    pp.col_scale = a->d_col_scale; pp.bias = a->d_bias;
    pp.absmax_out = a->d_absmax_out;
    pp.n_copies = a->n_out_copies;
    pp.copies_mc = a->out_copies_multicast != 0 ? 1 : 0;
    if (pp.copies_mc) {
        // only the row-wide store path has a multicast form: every tile must take it
        const bool two_byte = a->out_type == RNS_OUT_F16 || a->out_type == RNS_OUT_BF16;
        if (a->variant == 3 || a->n_out_copies != 1 || !two_byte || a->n % 128 != 0 || a->ldo % 8 != 0 ||
            (reinterpret_cast<uintptr_t>(a->d_out) & 15) || (reinterpret_cast<uintptr_t>(a->d_out_copies[0]) & 15))
            return fail(RNS_ERR_INVALID_ARGUMENT, "multicast output copies need variant 0/4, one copy address, two-byte "
                                                  "outputs, N %% 128 == 0, ldo %% 8 == 0 and 16-byte aligned bases");
    }
    for (int g = 0; g < a->n_out_copies && g < RNS_MAX_PEERS; ++g) {
        pp.out_copies[g] = a->d_out_copies[g];
        pp.absmax_copies[g] = a->d_absmax_copies[g];
    }
    pp.active = a->d_active_channels;
    pp.status = a->d_status; pp.wait_info = a->d_wait_info;
    const int64_t pairs = (int64_t)pp.n_ftiles * pp.n_ttiles * groups;
    if (pairs > (1 << 30)) return fail(RNS_ERR_UNSUPPORTED, "too many output tiles");
    if (a->d_absmax_out != nullptr) RNS_CUDA_OK(cudaMemsetAsync(a->d_absmax_out, 0, 2 * sizeof(uint32_t), st));
    // Variant 3 asks for the kernel that encodes canonical weight residues per channel;
    // otherwise every channel reads the int8 weight itself (same results, see
    // rns_gemm_pair_raw_sm100.cu).
    if (a->variant != 3) return launch_pair_raw_gemm(pp, (int)pairs, st);
    if (pp.n_copies > 0) {
        if (R == 4) return launch_pair<4, 128, 4, 6, true>(pp, (int)pairs, st);
        return launch_pair<5, 96, 4, 4, true>(pp, (int)pairs, st);
    }
    if (R == 4) return launch_pair<4, 128, 4, 6, false>(pp, (int)pairs, st);
    return launch_pair<5, 96, 4, 4, false>(pp, (int)pairs, st);
}

}  // namespace rns
