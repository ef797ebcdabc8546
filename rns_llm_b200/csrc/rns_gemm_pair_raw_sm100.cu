// Fused RNS linear for many-token calls on sm_100a, two CTAs per 256-feature x TOK-token
// tile (tcgen05 cta_group::2), with the int8 weight itself as the weight operand of
// every residue channel.
//
// Why that is the same result.  Channel c accumulates  S_c = sum_k a_c[k] * w_c[k]  and
// the epilogue uses only  S_c mod m_c.  Any representative of the weight's residue class
// gives the same S_c mod m_c, and the int8 value w is one (w = w_c mod m_c); what a
// canonical residue buys is a smaller |S_c|, which int32 accumulation does not need:
// |a_c| <= 128 and |w| <= 128 bound |S_c| by K * 2^14, inside int32 for every K the
// library accepts (K <= 131071, checked by the caller).  So the R weight tiles that
// rns_gemm_pair_sm100.cu encodes per K block collapse into ONE tile that a bulk copy
// brings from global memory as it lies; the activation residues stay per channel.
// Reconstructed integers, and everything after them, are bit-identical.
//
// What it changes on the SM: shared memory takes 8 KB of weights per K block and CTA
// instead of R x 8 KB written by sixteen encoder warps (whose stores shared the
// shared-memory data path with the MMA operand reads and held the tensor pipe near half
// of its rate), the ring is eight stages deep, and the sixteen warps only run epilogues.
//
// Per CTA: warp 18 lane 0 loads a stage (its 128 x 64 weight bytes and its half of the
// token tile's residue planes, R x TOK/2 x 64 bytes) onto one barrier; warps 0 and 1 of
// the leader CTA issue the MMAs of alternate stages; warp 1 of the peer CTA forwards
// "my half of the stage has landed"; warps 2..17 run the epilogue.  The first stage of a
// tile overwrites the accumulators (no zeroing pass); the warp that issues it tells the
// other issuer through a barrier before that one adds to them.  One tcgen05.commit per
// stage, multicast to both CTAs, releases the stage.  Every wait is bounded.
#include "rns_pair.cuh"

namespace rns {

#ifndef RNS_PAIR_SPLIT_EPILOGUE
#define RNS_PAIR_SPLIT_EPILOGUE 6   // two-phase epilogue up to this many channels (0: never), for comparison builds
#endif
// WCH: the weight operand is given per channel (R packed matrices, p.w_channel_stride
// bytes apart): sources wider than int8, whose residues do not fit the trick above, with
// the residue planes of the weight cached at prepare time.  S: ring depth (<= kDoneRing).
// ISSUERS: 2 = warps 0 and 1 take alternate stages (needs an even S, so that a slot keeps
// its warp and the warp sees every phase of the slot's barrier); 1 = warp 0 issues all.
// PREFIX: p.active points at the number of leading channels to compute (the adaptive
// prefix a preceding kernel chose on the device): the planes, MMAs and residues of the
// others are skipped, and the reconstruction uses the prefix's product.
template <int R, int TOK, int S, int ISSUERS, bool WCH, bool COPIES, bool PREFIX = false>
__global__ void __launch_bounds__(kPairThreads, 1)
rns_gemm_pair_raw_kernel(const __grid_constant__ PairParams p) {
    static_assert(!PREFIX || (!WCH && !COPIES), "the prefix form exists for one int8 weight matrix, no copies");
    static_assert(R * TOK <= 512, "accumulators must fit tensor memory");
    static_assert(TOK % 32 == 0 && (TOK / 2) % 8 == 0, "token tile shape");
    static_assert(S <= kDoneRing && (ISSUERS == 1 || (ISSUERS == 2 && S % 2 == 0)), "ring depth");
    constexpr int TR = TOK / 2;                               // token rows this CTA loads
    constexpr uint32_t kPlTile = (uint32_t)TR * kPackK;
    constexpr uint32_t kPlStage = (uint32_t)R * kPlTile;
    constexpr uint32_t kWStage = (WCH ? (uint32_t)R : 1u) * kPairOpTile;
    constexpr uint32_t kTmemCols = 512;

    extern __shared__ uint8_t smem_dyn[];
    __shared__ PairCtl ctl;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t tiles_base = (smem_addr(smem_dyn) + 1023u) & ~1023u;
    const uint32_t w_base = tiles_base;                        // weight ring first
    const uint32_t pl_base = tiles_base + (uint32_t)S * kWStage;

    const uint32_t rank = cluster_cta_rank();
    const int cluster = (int)(blockIdx.x >> 1), clusters = (int)(gridDim.x >> 1);
    const int tiles = p.n_ftiles * p.n_ttiles * (p.groups > 1 ? p.groups : 1);
    const int nst = p.kblocks;                                 // one K block of 64 bytes per stage
    const int my_tiles = (tiles - cluster + clusters - 1) / clusters;

    if (threadIdx.x == 0) {
        ctl.abort = 0;
        ctl.absmax = 0u;
        for (int s = 0; s < kDoneRing; ++s) {
            mbar_init(smem_addr(&ctl.full_op[s]), 1);          // unused here
            // leader: its own load and the peer's relay; peer: its own load
            mbar_init(smem_addr(&ctl.full_pl[s]), rank == 0 ? 2 : 1);
            mbar_init(smem_addr(&ctl.done[s]), 1);
        }
        mbar_init(smem_addr(&ctl.acc_full), ISSUERS);          // one commit from each issuer warp
        mbar_init(smem_addr(&ctl.tmem_free), 2 * kPairEncWarps);   // leader: both CTAs' epilogue warps
        mbar_init(smem_addr(&ctl.first_issued), 1);
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
    int act = R;                                               // every thread reads the same word
    if constexpr (PREFIX) act = min(max(*reinterpret_cast<const volatile int32_t*>(p.active), 1), R);

    if (warp == kPairPlaneWarp) {
        // ------------------------------ producer ----------------------------------
        if (lane == 0) {
            int g = 0;
            bool ok = true;
            for (int tile = cluster; tile < tiles && ok; tile += clusters) {
                const PairTile t = pair_tile<TOK>(p, tile, rank);
                const int8_t* pl_src = p.planes + ((int64_t)((t.grp * p.n_ttiles + t.tt) * 2 + (int)rank) * p.kblocks) * (int64_t)kPlStage;
                // Feature rows past the padded weight (possible only in the last tile's
                // second half) are not loaded; their outputs are never stored.
                const int64_t w_row0 = (int64_t)t.grp * p.w_group_rows + t.n0;    // first weight row of this CTA
                const bool w_rows = w_row0 < p.w_npad;
                const int8_t* w_src = p.w + w_row0 * kPackK;
                const int64_t kb_stride = p.w_npad * kPackK;
                const uint32_t pl_bytes = PREFIX ? (uint32_t)act * kPlTile : kPlStage;   // leading channels only
                const uint32_t bytes = pl_bytes + (w_rows ? kWStage : 0u);
                for (int st = 0; st < nst; ++st, ++g) {
                    if (g >= S &&
                        !wait_bounded<false, true>(smem_addr(&ctl.done[(g - S) & (kDoneRing - 1)]),
                                                   (uint32_t)((g - S) >> 3) & 1u, abort, wait_code(2, st))) {
                        ok = false;
                        break;
                    }
                    const int s = g % S;
                    const uint32_t bar = smem_addr(&ctl.full_pl[s]);
                    mbar_arrive_expect_tx(bar, bytes);
                    if (w_rows) {
#pragma unroll
                        for (int c = 0; c < (WCH ? R : 1); ++c)
                            bulk_load(w_base + (uint32_t)s * kWStage + (uint32_t)c * kPairOpTile,
                                      w_src + (int64_t)c * p.w_channel_stride + (int64_t)st * kb_stride, kPairOpTile, bar);
                    }
                    bulk_load(pl_base + (uint32_t)s * kPlStage, pl_src + (int64_t)st * kPlStage, pl_bytes, bar);
                }
            }
        }
        __syncwarp();
    } else if (warp <= 1) {
        const int total = my_tiles * nst;                      // stages this cluster runs
        if (rank == 0 && warp >= ISSUERS) {
            // the second warp has nothing to issue in the one-issuer form
        } else if (rank != 0) {
            // ------------------------------ relay (peer CTA) -----------------------
            // Tells the leader that this CTA's half of a stage has landed.  Loads run
            // several stages ahead of the MMAs, so this hop is off the critical path.
            if (warp == 1 && lane == 0) {
                for (int g = 0; g < total; ++g) {
                    if (!wait_bounded<false, true>(smem_addr(&ctl.full_pl[g % S]), (uint32_t)(g / S) & 1u, abort,
                                                   wait_code(4, g))) break;
                    mbar_arrive_remote_relaxed(smem_addr(&ctl.full_pl[g % S]), 0);
                }
            }
            __syncwarp();
        } else {
            // ------------------------------ MMA issuers (leader CTA) ---------------
            // Two warps take alternate stages (one warp's instruction stream per stage is
            // longer than its MMAs run).  Integer accumulation does not depend on the
            // order of the MMAs, except that the tile's first stage overwrites: the warp
            // that owns it issues it, then releases the other warp through first_issued.
            const uint32_t idesc = make_idesc(256u, (uint32_t)TOK);
            const uint64_t desc0 = make_smem_desc(0, kPackK);
            const uint32_t a_lo0 = w_base >> 4, b_lo0 = pl_base >> 4;
            bool ok = true;
            int g0 = 0;                                        // first stage of the current tile
            for (int ti = 0; ti < my_tiles && ok; ++ti, g0 += nst) {
                const bool owner = ISSUERS == 1 || ((g0 & 1) == warp);   // issues the tile's first stage
                // accumulators drained (by both CTAs) since the previous tile
                ok = warp_wait_bounded<false, true>(smem_addr(&ctl.tmem_free), (uint32_t)ti & 1u, abort, wait_code(9, ti));
                if (ok && !owner)
                    ok = warp_wait_bounded<false, true>(smem_addr(&ctl.first_issued), (uint32_t)ti & 1u, abort, wait_code(7, ti));
                if (!ok) break;
                tc_fence_after();
                for (int g = g0 + (ISSUERS == 2 ? ((g0 + warp) & 1) : 0); g < g0 + nst; g += ISSUERS) {
                    const int s = g % S;
                    ok = warp_wait_bounded<false, true>(smem_addr(&ctl.full_pl[s]), (uint32_t)(g / S) & 1u, abort, wait_code(6, g));
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t a_st = a_lo0 + (uint32_t)s * (kWStage >> 4);
                    const uint32_t b_st = b_lo0 + (uint32_t)s * (kPlStage >> 4);
                    const bool first = g == g0;
                    if (elect_one()) {
#pragma unroll
                        for (int c = 0; c < R; ++c) {
                            if (PREFIX && c >= act) continue;
#pragma unroll
                            for (int ks = 0; ks < 2; ++ks) {
                                const uint64_t da = desc0 | (uint64_t)(a_st + (WCH ? (uint32_t)c * (kPairOpTile >> 4) : 0u) + (uint32_t)ks * 2u);
                                const uint64_t db = desc0 | (uint64_t)(b_st + (uint32_t)c * (kPlTile >> 4) + (uint32_t)ks * 2u);
                                umma_i8_pair(tmem_base + (uint32_t)(c * TOK), da, db, idesc, (first && ks == 0) ? 0u : 1u);
                            }
                        }
                        umma_commit_pair(smem_addr(&ctl.done[g & (kDoneRing - 1)]));
                        if (first && ISSUERS == 2) {
                            tc_fence_before();
                            mbar_arrive(smem_addr(&ctl.first_issued));
                        }
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
        // ------------------------------ epilogue -----------------------------------
        const int quarter = warp & 3;                          // tensor-memory lanes 32*quarter .. +31
        const int part = (warp - 2) >> 2;                      // quarter of the token columns
        const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
        auto release = [&]() {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (rank == 0) mbar_arrive(smem_addr(&ctl.tmem_free));
                else mbar_arrive_remote_relaxed(smem_addr(&ctl.tmem_free), 0);
            }
        };
        release();                                             // nothing to drain before the first tile
        const bool is_float = p.out_type >= RNS_OUT_F16;
        const float rs_all = (is_float && p.row_scale_stride == 0) ? p.row_scale[0] : 0.0f;
        float biggest = 0.0f;
        int ti = 0;
        for (int tile = cluster; tile < tiles; tile += clusters, ++ti) {
            const PairTile t = pair_tile<TOK>(p, tile, rank);
            bool ok = warp_wait_bounded(smem_addr(&ctl.acc_full), (uint32_t)ti & 1u, abort, wait_code(11, ti));
            if constexpr (COPIES) {
                // The four warps of a token-column block meet at a barrier inside the epilogue
                // (row-wide stores): they enter it together or not at all, even when a wait
                // expires for one of them while the phase completes for another.
                int all;
                asm volatile("{\n\t.reg .pred pin, pout;\n\tsetp.ne.b32 pin, %1, 0;\n\t"
                             "bar.red.and.pred pout, %2, 128, pin;\n\tselp.b32 %0, 1, 0, pout;\n\t}"
                             : "=r"(all) : "r"(ok ? 1 : 0), "r"(2 + part) : "memory");
                ok = all != 0;
            }
            if (!ok) break;
            tc_fence_after();
            pair_epilogue<R, TOK, COPIES, (R <= 6 && R <= RNS_PAIR_SPLIT_EPILOGUE), PREFIX>(
                p, t.n0, t.tok0, quarter, part, lane, lane_base, is_float, rs_all, biggest, release,
                COPIES ? reinterpret_cast<unsigned short*>(smem_dyn + (tiles_base - smem_addr(smem_dyn)) +
                                                           (size_t)S * (kWStage + kPlStage)) : nullptr, act,
                (int64_t)t.grp * p.out_group_stride);
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
        const int total = my_tiles * nst;
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
                p.wait_info[3] = R * 1000000 + (WCH ? 400000 : 300000) + TOK;
            }
        } else if (p.absmax_out != nullptr) {
            if (ctl.absmax != 0u) atomicMax(p.absmax_out, ctl.absmax);
            if (COPIES && p.n_copies > 0) {
                // The last CTA to contribute hands the finished word to the other ranks.
                __threadfence();
                if (atomicAdd(p.absmax_out + 1, 1u) == gridDim.x - 1) {
                    const uint32_t final_word = atomicMax(p.absmax_out, 0u);
                    for (int g = 0; COPIES && g < p.n_copies; ++g) {
                        if (p.copies_mc) multimem_store_u32(p.absmax_copies[g], final_word);
                        else *p.absmax_copies[g] = final_word;
                    }
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
template <int R, int TOK, int S, int ISSUERS, bool WCH, bool COPIES, bool PREFIX = false>
static int launch_pair_raw(const PairParams& pp, int pairs, cudaStream_t st) {
    // COPIES: 16 KB behind the rings stage the row-wide stores (4 blocks x 2 buffers x 8 x 128 x 2 bytes)
    constexpr size_t smem = (size_t)S * ((WCH ? R : 1) * kPairOpTile + (size_t)R * (TOK / 2) * kPackK) + 1024 +
                            (COPIES ? kPairStageBytes : 0);
    static_assert(smem + sizeof(PairCtl) <= 227 * 1024, "ring exceeds shared memory");
    return launch_pair_clusters<rns_gemm_pair_raw_kernel<R, TOK, S, ISSUERS, WCH, COPIES, PREFIX>>(smem, pp, pairs, st);
}

int pair_raw_token_tile(int channels) { return channels <= 4 ? 128 : (channels == 5 ? 96 : 64); }

int launch_pair_raw_gemm(const PairParams& pp, int pairs, cudaStream_t st) {
    const int R = pp.plan.channels;
    if (pp.w_channel_stride != 0) {
        // residue planes of a wide weight: deeper stages, shallower rings; no output copies
        if (pp.n_copies > 0) return fail(RNS_ERR_UNSUPPORTED, "output copies are not built for per-channel weights");
        if (R == 4) return launch_pair_raw<4, 128, 4, 2, true, false>(pp, pairs, st);
        if (R == 5) return launch_pair_raw<5, 96, 4, 2, true, false>(pp, pairs, st);
        if (R == 6) return launch_pair_raw<6, 64, 3, 1, true, false>(pp, pairs, st);
        return fail(RNS_ERR_UNSUPPORTED, "per-channel weights: 4, 5 or 6 channels");
    }
    if (pp.active != nullptr) {
        if (pp.n_copies > 0) return fail(RNS_ERR_UNSUPPORTED, "an adaptive prefix and output copies are not built together");
        if (R == 4) return launch_pair_raw<4, 128, 8, 2, false, false, true>(pp, pairs, st);
        if (R == 5) return launch_pair_raw<5, 96, 8, 2, false, false, true>(pp, pairs, st);
        return fail(RNS_ERR_UNSUPPORTED, "adaptive prefix: 4 or 5 channels");
    }
    if (pp.n_copies > 0) {
        if (R == 4) return launch_pair_raw<4, 128, 8, 2, false, true>(pp, pairs, st);
        if (R == 5) return launch_pair_raw<5, 96, 8, 2, false, true>(pp, pairs, st);
        return fail(RNS_ERR_UNSUPPORTED, "output copies: 4 or 5 channels");
    }
    if (R == 4) return launch_pair_raw<4, 128, 8, 2, false, false>(pp, pairs, st);
    if (R == 5) return launch_pair_raw<5, 96, 8, 2, false, false>(pp, pairs, st);
    if (R == 6) return launch_pair_raw<6, 64, 8, 2, false, false>(pp, pairs, st);
    return fail(RNS_ERR_UNSUPPORTED, "the two-CTA kernel covers 4, 5 or 6 channels");
}

}  // namespace rns
