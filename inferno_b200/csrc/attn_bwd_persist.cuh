// Causal flash-attention backward for sm_100a: persistent CTAs (bf16 operands, and fp32 I/O carried as hi/lo bf16 pairs).
//
// Block algorithm, warp roles, shared-memory and TMEM plan: attn_bwd.cuh (which names the reference nodes the backward
// replaces).  One CTA per SM walks a list of work items (one item = one 128-row key / value tile of one head), and all
// mbarrier phases run on from item to item (each role counts the query blocks it has handled), so that
//   * the TMA warp loads the next item's K and V tiles as soon as the last MMA of the current item has completed, and
//     keeps the Q / dO ring running straight into the next item;
//   * the four drain warps, not the compute warps, turn dK / dV into bf16 (staged in their own dQ^T staging tile, which
//     has the size of one bf16 dK / dV tile) and store them, so the compute warps go straight on to the next item's first
//     blocks and the MMA warp to its S^T / dP^T / dQ^T; only an item's first dK / dV MMAs wait until the drain warps have
//     read the accumulators out of TMEM;
//   * a CTA's launch, barrier set-up, TMEM allocation and tear-down are paid once per SM instead of once per item.
// A CTA launched per item spends about 11 us outside its steady state (17 % of an average item at T = 4096; measured
// on the one-CTA-per-item form this kernel replaced).
// Items are drawn, not assigned: a CTA starts on item blockIdx.x and its TMA thread draws every further index from a
// counter in global memory (ItemRing in sm100_ptx.cuh hands it to the other roles).  The list runs over groups of
// consecutive heads (locate_item) so that the CTAs share the Q / dO tiles and the fp32 dQ accumulator of few heads in L2 at
// a time, and inside a group from key tile 0 (the longest walk) to the last.
#pragma once

#include "attn_bwd.cuh"

namespace ib200 {

template <class TR>
__global__ void __launch_bounds__(TR::THREADS, 1)
attn_bwd_persist_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_q_lo,
                        const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_k_lo,
                        const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_v_lo,
                        const __grid_constant__ CUtensorMap tm_do, const __grid_constant__ CUtensorMap tm_do_lo,
                        const __grid_constant__ CUtensorMap tm_dk, const __grid_constant__ CUtensorMap tm_dv,
                        const __grid_constant__ CUtensorMap tm_dq, BwdParams prm, int n_items, int n_groups, int* next_item) {
    constexpr int D = TR::D, BKV = TR::BKV, BQ = TR::BQ, NS = TR::NS, NB = TR::NB;
    constexpr bool SPLIT = TR::SPLIT;
    // groups of four queries (of the eight a compute thread handles per block) whose lse / delta values are fetched early;
    // measured on one GPU with the builds swapped in place: at D = 128 all 8 (+2 % at T >= 4096 over 6, -2.5 % at T = 1024), at
    // D = 64 4 (6 and 8 cost 3-12 %: the variant starts to spill)
    // (split mode: none -- its compute threads carry twice the packed values, and early loads made them spill)
    constexpr int kPre = SPLIT ? 0 : (D == 128) ? 8 : 4;
    constexpr int kPreN = kPre > 0 ? kPre : 1;
    // D = 128: wait for the dS^T tile before phase two instead of just before the stores (+0.5-1 %; -3 % at D = 64)
    constexpr bool kWaitDsEarly = (D == 128);
    // D = 64: S^T is handed to the compute warps before dP^T has been issued, so that their exponentials run under it (+8 %);
    // at D = 128, where the MMA side paces the block, the extra commit and wait bought nothing and one hand-off is used
    // (split mode triples the MMA work per block, so there too the MMA side paces and one hand-off is used)
    constexpr bool kSplitHandoff = (D == 64) && !SPLIT;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint8_t* sK = smem + TR::OFF_K;
    uint8_t* sV = smem + TR::OFF_V;
    uint8_t* sQ = smem + TR::OFF_Q;
    uint8_t* sDO = smem + TR::OFF_DO;
    uint8_t* sDS = smem + TR::OFF_DS;
    float* sVec = reinterpret_cast<float*>(smem + TR::OFF_VEC);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + TR::OFF_BAR);
    uint64_t* kv_full = bars;               // [1]   K, V of an item
    uint64_t* qdo_full = bars + 1;          // [NS]  TMA: Q, dO tiles + staged lse/delta
    uint64_t* qdo_empty = qdo_full + NS;    // [NS]  MMA commit: block consumed
    uint64_t* sdp_full = qdo_empty + NS;    // [NB]  MMA commit: S^T of a block is in TMEM (dP^T follows: dp_full)
    uint64_t* pds_full = sdp_full + NB;     // [NB]  compute warps: P^T, dS^T written (TMEM + smem)
    uint64_t* dq_full = pds_full + NB;      // [NB]  MMA commit: dQ^T in TMEM (and the dS^T smem tile is free)
    uint64_t* dq_empty = dq_full + NB;      // [NB]  drain warps: dQ^T copied to registers
    uint64_t* dkv_full = dq_empty + NB;     // [1]   MMA commit: every MMA of the item has completed (dK, dV final; K, V tiles free)
    uint64_t* dkv_free = dkv_full + 1;      // [1]   drain warps (4): dK, dV read out of TMEM
    uint64_t* dp_full = dkv_free + 1;       // [NB]  MMA commit: dP^T of a block is in TMEM
    uint64_t* item_bars = dp_full + NB;     // [4]   item ring: full[2], empty[2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(item_bars + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const ItemRing items{item_bars, item_bars + 2, abort_flag + 1};

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int T = prm.T;
    const int BH = prm.BH;
    const int nqb = (T + BQ - 1) / BQ;
    const int n_kt = (T + BKV - 1) / BKV;
    AbortCtx ab{abort_flag, prm.status};

    // item -> head, key tile, first query block, number of query blocks (identical in every role)
    struct Item { int bh, hd, bt, n, m0, nblk; };
    auto decode = [&](int idx) {
        Item it;
        locate_item(HeadGroups{BH, n_groups, n_kt}, idx, it.n, it.bh);   // key tile 0 walks the most query blocks: first
        it.hd = it.bh % prm.H;
        it.bt = it.bh / prm.H;
        it.m0 = prm.causal ? (it.n * BKV) / BQ : 0;                 // first query block at or below the diagonal
        it.nblk = nqb - it.m0;
        return it;
    };

    if (tid == 0) {
        *abort_flag = 0;
        mbar_init(kv_full, 1);
        for (int s = 0; s < NS; ++s) { mbar_init(&qdo_full[s], 1); mbar_init(&qdo_empty[s], 1); }
        for (int b = 0; b < NB; ++b) {
            mbar_init(&sdp_full[b], 1); mbar_init(&dp_full[b], 1); mbar_init(&pds_full[b], 8);
            mbar_init(&dq_full[b], 1); mbar_init(&dq_empty[b], 4);
        }
        mbar_init(dkv_full, 1);
        mbar_init(dkv_free, 4);
        item_ring_init(items, 13);               // readers: the MMA warp, eight compute warps, four drain warps
        fence_mbar_init();
    }
    if (warp == 13) { tmem_alloc(tmem_slot, TR::TM_COLS); tmem_relinquish(); }
    if (warp == 12 && lane == 0) {
        tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_k); tma_prefetch_desc(&tm_v); tma_prefetch_desc(&tm_do);
        tma_prefetch_desc(&tm_dk); tma_prefetch_desc(&tm_dv); tma_prefetch_desc(&tm_dq);
        if constexpr (SPLIT) { tma_prefetch_desc(&tm_q_lo); tma_prefetch_desc(&tm_k_lo); tma_prefetch_desc(&tm_v_lo); tma_prefetch_desc(&tm_do_lo); }
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    if (warp >= 12) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 80;");
    } else if (warp >= 8) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 112;");
    }

    if (warp == 12) {
        // ------------------------------ producer ------------------------------
        if (lane == 0) {
            uint32_t g = 0;                                         // query blocks loaded so far (ring position and phase)
            int ni = 0;
            for (int idx = blockIdx.x; idx < n_items; ++ni) {
                if (*abort_flag != 0) break;
                const Item item = decode(idx);
                // draw the next item now; the value is needed (and published to the other roles) only after this item's K / V loads
                const int drawn = atomicAdd(next_item, 1);
                if (ni > 0) mbar_wait(dkv_full, (ni - 1) & 1, ab, 12);          // the previous item's MMAs have finished with K, V
                mbar_arrive_expect_tx(kv_full, 2 * TR::KV_TILE);
                // panel p of a tile: columns 64p.. of a bf16 operand, or (fp32 I/O) the hi / lo half of the bf16 pair
                auto col = [](int p) { return SPLIT ? 0 : p * 64; };
                for (int p = 0; p < TR::NP; ++p) {
                    tma_load_4d(sK + p * TR::KV_PANEL, (SPLIT && p) ? &tm_k_lo : &tm_k, kv_full, col(p), item.n * BKV, item.hd, item.bt);
                    tma_load_4d(sV + p * TR::KV_PANEL, (SPLIT && p) ? &tm_v_lo : &tm_v, kv_full, col(p), item.n * BKV, item.hd, item.bt);
                }
                idx = static_cast<int>(gridDim.x) + drawn;
                item_ring_publish(items, ni, idx, ab);
                for (int it = 0; it < item.nblk; ++it, ++g) {
                    const int s = g % NS;
                    const int m = item.m0 + it;
                    mbar_wait(&qdo_empty[s], ((g / NS) & 1) ^ 1, ab, 10);
                    mbar_arrive_expect_tx(&qdo_full[s], 2 * TR::Q_TILE + 2 * BQ * 4);
                    for (int p = 0; p < TR::NP; ++p) {
                        tma_load_4d(sQ + s * TR::Q_TILE + p * TR::Q_PANEL, (SPLIT && p) ? &tm_q_lo : &tm_q, &qdo_full[s], col(p), m * BQ, item.hd, item.bt);
                        tma_load_4d(sDO + s * TR::Q_TILE + p * TR::Q_PANEL, (SPLIT && p) ? &tm_do_lo : &tm_do, &qdo_full[s], col(p), m * BQ, item.hd, item.bt);
                    }
                    // the block's 64 values of -lse*log2e and of -delta (padded rows, so always aligned and in range)
                    const size_t voff = static_cast<size_t>(item.bh) * prm.T_pad + static_cast<size_t>(m) * BQ;
                    bulk_load_1d(sVec + s * 2 * BQ, prm.nlse2 + voff, BQ * 4, &qdo_full[s]);
                    bulk_load_1d(sVec + s * 2 * BQ + BQ, prm.ndelta + voff, BQ * 4, &qdo_full[s]);
                }
            }
        }
    } else if (warp == 13) {
        // ------------------------------ MMA issuer (converged warp, one elected lane issues) ------------------------------
        const bool leader = elect_one_lane();
        // descriptor low words: K-major views (lbo unused = 16) and MN-major views (lbo = panel stride)
        const uint32_t lK = sdesc_lo(smem_u32(sK), 16), lV = sdesc_lo(smem_u32(sV), 16);
        const uint32_t lK_mn = sdesc_lo(smem_u32(sK), TR::KV_PANEL), lDS = sdesc_lo(smem_u32(sDS), 16);
        const uint32_t lQ0 = sdesc_lo(smem_u32(sQ), 16), lDO0 = sdesc_lo(smem_u32(sDO), 16);
        constexpr uint32_t kStage = TR::Q_TILE >> 4;                               // ring stage stride in descriptor units
        constexpr uint32_t kToMN = ((TR::Q_PANEL >> 4) << 16) - (1u << 16);        // K-major view -> MN-major view of a Q/dO stage
        // S^T and dP^T of global block gb into buffer gb % NB; the dP^T buffer must have been drained of dQ^T(gb - NB)
        auto issue_front = [&](uint32_t gb) {
            const uint32_t b = gb % NB, s = gb % NS;
            mbar_wait(&qdo_full[s], (gb / NS) & 1, ab, 21);
            tc_fence_after_sync();
            bwd_issue_kmajor<TR>(tmem + TR::TM_ST + b * 64, lK, lQ0 + s * kStage, leader);
            if (kSplitHandoff && leader) umma_commit(&sdp_full[b]);    // the compute warps start on the exponentials while dP^T is still to come
            if (gb >= NB) { mbar_wait(&dq_empty[b], ((gb - NB) / NB) & 1, ab, 24); tc_fence_after_sync(); }
            bwd_issue_kmajor<TR>(tmem + TR::TM_DP + b * 64, lV, lDO0 + s * kStage, leader);
            if (leader) umma_commit(kSplitHandoff ? &dp_full[b] : &sdp_full[b]);
        };
        uint32_t g0 = 0;                                                            // global index of the item's first block
        int ni = 0;
        for (int idx = blockIdx.x; idx < n_items; idx = item_ring_next(items, ni++, ab, leader)) {
            if (*abort_flag != 0) break;
            const Item item = decode(idx);
            const int nblk = item.nblk;
            mbar_wait(kv_full, ni & 1, ab, 20);
#pragma unroll
            for (int j = 0; j < NB; ++j)
                if (j < nblk) issue_front(g0 + j);
            for (int it = 0; it < nblk; ++it) {
                const uint32_t gb = g0 + it;
                const uint32_t b = gb % NB, s = gb % NS;
                const uint32_t lQ_mn = lQ0 + s * kStage + kToMN, lDO_mn = lDO0 + s * kStage + kToMN;
                const uint32_t t_st = tmem + TR::TM_ST + b * 64, t_dp = tmem + TR::TM_DP + b * 64;
                mbar_wait(&pds_full[b], (gb / NB) & 1, ab, 22);
                tc_fence_after_sync();
                if constexpr (!SPLIT) {
                    bwd_issue_dq<TR>(t_dp, lK_mn, lDS, leader);                            // dQ^T over the consumed dP^T buffer
                    if (leader) umma_commit(&dq_full[b]);
                    // the item's first dK / dV MMAs overwrite the accumulators: the previous epilogue must have read them
                    if (it == 0 && ni > 0) { mbar_wait(dkv_free, (ni - 1) & 1, ab, 26); tc_fence_after_sync(); }
                    bwd_issue_acc<TR>(tmem + TR::TM_DK, t_st, 1, lQ_mn, it > 0, leader);   // dK += dS^T Q
                    bwd_issue_acc<TR>(tmem + TR::TM_DV, t_st, 0, lDO_mn, it > 0, leader);  // dV += P^T dO
                } else {
                    // split mode: {P^T hi, lo} live in the S^T buffer and {dS^T hi, lo} in the dP^T buffer, so dK reads the
                    // latter before dQ^T overwrites it
                    if (it == 0 && ni > 0) { mbar_wait(dkv_free, (ni - 1) & 1, ab, 26); tc_fence_after_sync(); }
                    bwd_issue_acc<TR>(tmem + TR::TM_DV, t_st, 0, lDO_mn, it > 0, leader);
                    bwd_issue_acc<TR>(tmem + TR::TM_DK, t_dp, 0, lQ_mn, it > 0, leader);
                    bwd_issue_dq<TR>(t_dp, lK_mn, lDS, leader);
                    if (leader) umma_commit(&dq_full[b]);
                }
                if (leader) umma_commit(&qdo_empty[s]);
                if (it + NB < nblk) issue_front(gb + NB);
            }
            if (leader) umma_commit(dkv_full);
            g0 += nblk;
        }
    } else if (warp < 8) {
        // ------------------------------ compute: P^T and dS^T ------------------------------
        asm volatile("setmaxnreg.inc.sync.aligned.u32 160;");
        const int h = warp >> 2;                     // which 32 query columns
        const int wq = warp & 3;
        const int r = wq * 32 + lane;                // key row inside the tile
        const uint32_t lane_base = static_cast<uint32_t>(wq * 32) << 16;
        const float c = prm.scale_log2;
        uint32_t g0 = 0;
        int ni = 0;
        for (int idx = blockIdx.x; idx < n_items; idx = item_ring_next(items, ni++, ab, lane == 0)) {
            if (*abort_flag != 0) break;
            const Item item = decode(idx);
            const int n = item.n, m0 = item.m0, nblk = item.nblk;
            const int kv_g = n * BKV + r;
            const bool row_dead = kv_g >= T;
            const bool tail_tile = (n + 1) * BKV > T;     // this key tile has rows past T

            for (int it = 0; it < nblk; ++it) {
                const uint32_t gb = g0 + it;
                const int b = gb % NB, s = gb % NS, m = m0 + it;
                const float* v_lse = sVec + s * 2 * BQ + h * 32;
                const float* v_del = v_lse + BQ;
                const uint32_t t_st = tmem + TR::TM_ST + b * 64 + h * 32 + lane_base;
                const uint32_t t_dp = tmem + TR::TM_DP + b * 64 + h * 32 + lane_base;
                mbar_wait(&qdo_full[s], (gb / NS) & 1, ab, 30);      // lse / delta visible
                // the block's -lse*log2e and -delta values (kPre groups of four queries) now, under the wait for S^T / dP^T: with
                // the MMA operand reads loading the shared-memory pipe these broadcast loads take a few hundred cycles when
                // issued in the element loop
                float4 nl_pre[kPreN], nd_pre[kPreN];
#pragma unroll
                for (int e4 = 0; e4 < kPre; ++e4) {
                    nl_pre[e4] = reinterpret_cast<const float4*>(v_lse)[e4];
                    nd_pre[e4] = reinterpret_cast<const float4*>(v_del)[e4];
                }
                mbar_wait(&sdp_full[b], (gb / NB) & 1, ab, 31);
                tc_fence_after_sync();
                uint32_t sr[32], dr[32];
                tmem_ld_x32(t_st, sr);
                tmem_wait_ld();
                const bool diag = prm.causal && (m * BQ < (n + 1) * BKV);
                const int q0 = m * BQ + h * 32;
                const bool masked = diag || tail_tile;             // uniform per block: most blocks take the unmasked path
                uint32_t pk[16], dk[16], pl[16], dl[16];       // (hi, lo) bf16 pairs; the lo halves only in split mode
                const uint64_t c2 = pack_f32x2(c, c);
                const float4* v_lse4 = reinterpret_cast<const float4*>(v_lse);
                const float4* v_del4 = reinterpret_cast<const float4*>(v_del);
                // Phase one, as soon as S^T is there: P^T = exp2(c S^T - lse), kept in sr as fp32 bits and packed to bf16.
                // The masked and the unmasked block are two copies of the loop: a branch inside the loop body would cut it
                // into one basic block per element pair and expose the full FFMA -> MUFU -> convert latency 16 times.
                auto body_p = [&](auto masked_tag) {
                    constexpr bool kMasked = decltype(masked_tag)::value;
#pragma unroll
                    for (int e4 = 0; e4 < 8; ++e4) {
                        const float4 nl = e4 < kPre ? nl_pre[e4 < kPre ? e4 : 0] : v_lse4[e4];   // broadcast 16-byte loads: 4 query columns each
#pragma unroll
                        for (int half = 0; half < 2; ++half) {
                            const int e = e4 * 4 + half * 2;
                            const uint64_t nl2 = half ? pack_f32x2(nl.z, nl.w) : pack_f32x2(nl.x, nl.y);
                            float x0, x1;
                            unpack_f32x2(ffma2(pack_f32x2(__uint_as_float(sr[e]), __uint_as_float(sr[e + 1])), c2, nl2), x0, x1);
                            float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
                            if constexpr (kMasked) {
                                if (row_dead || (diag && kv_g > q0 + e)) p0 = 0.f;
                                if (row_dead || (diag && kv_g > q0 + e + 1)) p1 = 0.f;
                            }
                            sr[e] = __float_as_uint(p0);
                            sr[e + 1] = __float_as_uint(p1);
                            pk[e >> 1] = pack_bf16x2(p0, p1);
                            if constexpr (SPLIT)
                                pl[e >> 1] = pack_bf16x2(p0 - __uint_as_float(pk[e >> 1] << 16), p1 - __uint_as_float(pk[e >> 1] & 0xffff0000u));
                        }
                    }
                };
                if (masked) body_p(MaskedTag<true>{}); else body_p(MaskedTag<false>{});
                tmem_st_x16(t_st, pk);
                if constexpr (SPLIT) tmem_st_x16(t_st + 16, pl);
                // Phase two, once dP^T is there: dS^T = P^T o (dP^T - delta).
                // The single dS^T shared-memory tile is free once dQ^T of the previous block (of this or the previous item) has
                // completed (a second tile was measured at both head dims: no gain at D = 128, +2 % at D = 64 and T = 8192 but
                // -1 % at T <= 1024); at D = 128 that wait comes first.
                if (kWaitDsEarly && gb >= 1) mbar_wait(&dq_full[(gb - 1) % NB], ((gb - 1) / NB) & 1, ab, 32);
                if constexpr (kSplitHandoff) {
                    mbar_wait(&dp_full[b], (gb / NB) & 1, ab, 34);
                    tc_fence_after_sync();
                }
                tmem_ld_x32(t_dp, dr);
                tmem_wait_ld();
#pragma unroll
                for (int e4 = 0; e4 < 8; ++e4) {
                    const float4 nd = e4 < kPre ? nd_pre[e4 < kPre ? e4 : 0] : v_del4[e4];
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        const int e = e4 * 4 + half * 2;
                        const uint64_t nd2 = half ? pack_f32x2(nd.z, nd.w) : pack_f32x2(nd.x, nd.y);
                        const uint64_t p2 = pack_f32x2(__uint_as_float(sr[e]), __uint_as_float(sr[e + 1]));
                        float d0, d1;
                        unpack_f32x2(fmul2(p2, fadd2(pack_f32x2(__uint_as_float(dr[e]), __uint_as_float(dr[e + 1])), nd2)), d0, d1);
                        dk[e >> 1] = pack_bf16x2(d0, d1);
                        if constexpr (SPLIT)
                            dl[e >> 1] = pack_bf16x2(d0 - __uint_as_float(dk[e >> 1] << 16), d1 - __uint_as_float(dk[e >> 1] & 0xffff0000u));
                    }
                }
                if constexpr (!SPLIT) {
                    tmem_st_x16(t_st + 16, dk);
                } else {
                    tmem_st_x16(t_dp, dk);          // dP^T has been read into registers: its buffer takes {dS^T hi, lo}
                    tmem_st_x16(t_dp + 16, dl);
                }
                if (!kWaitDsEarly && gb >= 1) mbar_wait(&dq_full[(gb - 1) % NB], ((gb - 1) / NB) & 1, ab, 32);
#pragma unroll
                for (int c4 = 0; c4 < 4; ++c4) {
                    st_shared_sw128(sDS, r, h * 4 + c4, make_uint4(dk[4 * c4], dk[4 * c4 + 1], dk[4 * c4 + 2], dk[4 * c4 + 3]));
                    if constexpr (SPLIT)
                        st_shared_sw128(sDS + TR::DS_PART, r, h * 4 + c4, make_uint4(dl[4 * c4], dl[4 * c4 + 1], dl[4 * c4 + 2], dl[4 * c4 + 3]));
                }
                tmem_wait_st();
                fence_proxy_async_smem();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(&pds_full[b]);
            }
            g0 += nblk;
        }
    } else if (warp < 12) {
        // ------------------------------ drain dQ^T ------------------------------
        const int wq = warp & 3;
        const uint32_t lane_base = static_cast<uint32_t>(wq * 32) << 16;
        // M = D rows of dQ^T: D=128 fills all lanes; D=64 uses lanes 0-15 of each quarter
        const int d = (D == 128) ? (wq * 32 + lane) : (wq * 16 + lane);
        const bool lane_ok = (D == 128) || (lane < 16);
        float* stage = reinterpret_cast<float*>(smem + TR::OFF_DQ);
        const bool issuer = (tid == 256);
        uint32_t g0 = 0;
        for (int nd = 0, idx = blockIdx.x; idx < n_items; idx = item_ring_next(items, nd++, ab, lane == 0)) {
            if (*abort_flag != 0) break;
            const Item item = decode(idx);
            for (int it = 0; it < item.nblk; ++it) {
                const uint32_t gb = g0 + it;
                const int b = gb % NB, m = item.m0 + it;
                mbar_wait(&dq_full[b], (gb / NB) & 1, ab, 40);
                tc_fence_after_sync();
                uint32_t r0[32], r1[32];
                tmem_ld_x32(tmem + TR::TM_DP + b * 64 + lane_base, r0);
                tmem_ld_x32(tmem + TR::TM_DP + b * 64 + 32 + lane_base, r1);
                tmem_wait_ld();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(&dq_empty[b]);
                // the previous block's reduction must have finished reading the staging tile
                if (issuer) tma_store_wait_read_all();
                asm volatile("bar.sync 3, 128;" ::: "memory");
                if (lane_ok) {
#pragma unroll
                    for (int e = 0; e < 32; ++e) stage[e * D + d] = SPLIT ? __uint_as_float(r0[e]) * prm.dq_scale : __uint_as_float(r0[e]);
#pragma unroll
                    for (int e = 0; e < 32; ++e) stage[(32 + e) * D + d] = SPLIT ? __uint_as_float(r1[e]) * prm.dq_scale : __uint_as_float(r1[e]);
                }
                fence_proxy_async_smem();
                asm volatile("bar.sync 3, 128;" ::: "memory");
                if (issuer) {
                    tma_reduce_add_3d(&tm_dq, stage, 0, m * BQ, item.bh);    // rows past T are clipped
                    tma_store_commit();
                }
            }
            g0 += item.nblk;

            // ---- epilogue of the item: dV, then dK (scaled), one key row per thread, staged as bf16 in the dQ^T staging tile
            // (same size) and stored by TMA.  The compute warps are already on the next item's first blocks.
            mbar_wait(dkv_full, nd & 1, ab, 41);
            tc_fence_after_sync();
            const int r = wq * 32 + lane;
            uint8_t* stage_b = reinterpret_cast<uint8_t*>(stage);
#pragma unroll
            for (int hsel = 0; hsel < 2; ++hsel) {
                const uint32_t t_acc = tmem + (hsel ? TR::TM_DK : TR::TM_DV) + lane_base;
                const float mul = hsel ? prm.scale : 1.f;
                if (issuer) tma_store_wait_read_all();           // the previous reduction / store has read the staging tile
                asm volatile("bar.sync 3, 128;" ::: "memory");
#pragma unroll
                for (int cc = 0; cc < D; cc += 32) {
                    uint32_t rr[32];
                    tmem_ld_x32(t_acc + cc, rr);
                    tmem_wait_ld();
                    if (hsel == 1 && cc + 32 == D) {
                        // dK / dV are in registers or staged: the next item's first dK / dV MMAs may overwrite the accumulators
                        tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(dkv_free);
                    }
                    if constexpr (!SPLIT) {
                        const int panel = cc / 64, chunk0 = (cc % 64) / 8;
#pragma unroll
                        for (int q4 = 0; q4 < 4; ++q4) {
                            uint4 v;
                            v.x = pack_bf16x2(__uint_as_float(rr[q4 * 8 + 0]) * mul, __uint_as_float(rr[q4 * 8 + 1]) * mul);
                            v.y = pack_bf16x2(__uint_as_float(rr[q4 * 8 + 2]) * mul, __uint_as_float(rr[q4 * 8 + 3]) * mul);
                            v.z = pack_bf16x2(__uint_as_float(rr[q4 * 8 + 4]) * mul, __uint_as_float(rr[q4 * 8 + 5]) * mul);
                            v.w = pack_bf16x2(__uint_as_float(rr[q4 * 8 + 6]) * mul, __uint_as_float(rr[q4 * 8 + 7]) * mul);
                            st_shared_sw128(stage_b + panel * TR::KV_PANEL, r, chunk0 + q4, v);
                        }
                    } else {
                        const int panel = cc / 32;     // 32 fp32 columns = one 128-byte panel row
#pragma unroll
                        for (int q4 = 0; q4 < 8; ++q4) {
                            uint4 v;
                            v.x = __float_as_uint(__uint_as_float(rr[q4 * 4 + 0]) * mul);
                            v.y = __float_as_uint(__uint_as_float(rr[q4 * 4 + 1]) * mul);
                            v.z = __float_as_uint(__uint_as_float(rr[q4 * 4 + 2]) * mul);
                            v.w = __float_as_uint(__uint_as_float(rr[q4 * 4 + 3]) * mul);
                            st_shared_sw128(stage_b + panel * TR::KV_PANEL, r, q4, v);
                        }
                    }
                }
                fence_proxy_async_smem();
                asm volatile("bar.sync 3, 128;" ::: "memory");
                if (issuer) {
                    for (int p = 0; p < TR::OUT_PANELS; ++p)
                        tma_store_4d(hsel ? &tm_dk : &tm_dv, stage_b + p * TR::KV_PANEL, p * TR::OUT_PANEL_ELEMS, item.n * BKV, item.hd, item.bt);
                    tma_store_commit();
                }
            }
        }
        if (issuer) tma_store_wait_read_all();
    }

    // ------------------------------ tear-down ------------------------------
    tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag != 0) {
        for (int it = 0; it < 64; ++it) __nanosleep(1000);
    }
    if (warp == 13) tmem_dealloc(tmem, TR::TM_COLS);
}

}  // namespace ib200
