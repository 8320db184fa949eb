// Causal flash-attention forward for sm_100a: persistent CTAs (bf16 operands, and fp32 I/O carried as hi/lo bf16 pairs).
//
// Tile algorithm, warp roles and TMEM plan: attn_fwd.cuh (which names the reference code the forward replaces:
// InfernoApp/main.cpp:737-754).  Outer structure: one CTA per SM walks a list of work items (one item = two adjacent
// 128-row query tiles of one head), and the roles run ahead of each other across item boundaries:
//   * the TMA warp loads the next item's Q tiles and first K tile as soon as the last S = Q K^T of the current item has
//     been issued and completed (barrier q_free), i.e. during the current item's last key tile and epilogue;
//   * the MMA warp issues the next item's first S MMAs as soon as those tiles have landed, under the epilogue;
//   * O is staged for its TMA store in a tile of its own (not in the Q tiles), and the next item's first P.V waits only
//     until the epilogue has read O out of TMEM (barrier o_free).
// A CTA launched per item pays about 7 us for launch, the first loads, the pipeline fill and the epilogue (measured on
// the one-CTA-per-item form this kernel replaced): 20 % of an average item at T = 4096 and half of one at T = 1024;
// here most of it runs under another item's work.
// All mbarrier phases run on from item to item; each role derives them from its own counters.
// Items are drawn, not assigned: a CTA starts on item blockIdx.x and its TMA thread draws every further index from a
// counter in global memory (ItemRing in sm100_ptx.cuh hands it to the other roles), so CTAs that drew short walks draw more
// of them.  The list runs over groups of consecutive heads (locate_item) so that the CTAs share the K / V tiles of few
// heads in L2 at a time, and inside a group from the longest walk to the shortest.
#pragma once

#include "attn_fwd.cuh"

namespace ib200 {

template <int D_, bool SPLIT_ = false>
struct FwdPersistTraits : FwdTraits<D_, SPLIT_> {
    using Base = FwdTraits<D_, SPLIT_>;
    static constexpr int OFF_STAGE = Base::SMEM_TILES * Base::TILE_BYTES;      // one O staging tile, used by both query tiles in turn
    static constexpr int OFF_BAR = OFF_STAGE + Base::TILE_BYTES;
    static constexpr int SMEM_BYTES = OFF_BAR + 512 + 1024 /*align slack*/;
    static_assert(SMEM_BYTES <= 232448, "shared memory budget");
};

struct FwdPersistParams {
    FwdParams p;
    int n_items;        // pairs_per_head * BH
    int pairs_per_head; // ceil(T / 256)
    int n_groups;       // head groups of the item list (see locate_item)
    int* next_item;     // draw counter in global memory, zero at launch
};

template <class TR>
__global__ void __launch_bounds__(TR::THREADS, 1)
attn_fwd_persist_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_q_lo,
                        const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_k_lo,
                        const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_v_lo,
                        const __grid_constant__ CUtensorMap tm_o, FwdPersistParams pp) {
    constexpr int D = TR::D, BM = TR::BM, BN = TR::BN, KS = TR::KV_STAGES;
    const FwdParams& prm = pp.p;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint8_t* sQ = smem;                                   // 2 tiles
    uint8_t* sK = sQ + 2 * TR::TILE_BYTES;                // KS tiles
    uint8_t* sV = sK + KS * TR::TILE_BYTES;               // KS tiles
    uint8_t* sO = smem + TR::OFF_STAGE;                   // O staging
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + TR::OFF_BAR);
    uint64_t* q_full = bars;                // [1]   query tiles + K_0 of an item
    uint64_t* q_free = bars + 1;            // [1]   every S MMA of an item has completed: Q tiles and all K slots are free
    uint64_t* k0_free = bars + 2;           // [1]   the first S MMAs of an item have read K_0
    uint64_t* kv_full = bars + 3;           // [KS]  load group: K_{j+1} and V_j
    uint64_t* kv_empty = kv_full + KS;      // [KS]
    uint64_t* s_full = kv_empty + KS;       // [2]   S_i is in TMEM (and every MMA issued before it has completed)
    uint64_t* p_half = s_full + 2;          // [2][2]  P columns 0-63 / 64-127 of tile i are in TMEM
    uint64_t* o_full = p_half + 4;          // [2]   after the last P.V of tile i of an item
    uint64_t* o_free = o_full + 2;          // [2]   the epilogue has read O_i out of TMEM (4 warps)
    uint64_t* stage_free = o_free + 2;      // [1]   the TMA store has read the staging tile
    uint64_t* ring_bars = stage_free + 1;   // [4]   item ring: full[2], empty[2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ring_bars + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const ItemRing ring{ring_bars, ring_bars + 2, abort_flag + 1};

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int T = prm.T;
    const int BH = prm.BH;
    const int n_kv_total = (T + BN - 1) / BN;
    AbortCtx ab{abort_flag, prm.status};

    // item -> head, query tiles, key-tile counts (identical in every role)
    struct Item { int bh, hd, bt, m0, m1, nkv0, nkv1, n_iter; };
    auto decode = [&](int idx) {
        Item it;
        int rank;
        locate_item(HeadGroups{BH, pp.n_groups, pp.pairs_per_head}, idx, rank, it.bh);
        const int pair = pp.pairs_per_head - 1 - rank;            // the last pair walks the most key tiles: first
        it.hd = it.bh % prm.H;
        it.bt = it.bh / prm.H;
        it.m0 = 2 * pair;
        it.m1 = 2 * pair + 1;
        const bool v0 = it.m0 * BM < T, v1 = it.m1 * BM < T;
        it.nkv0 = !v0 ? 0 : (prm.causal ? min(it.m0 + 1, n_kv_total) : n_kv_total);
        it.nkv1 = !v1 ? 0 : (prm.causal ? min(it.m1 + 1, n_kv_total) : n_kv_total);
        it.n_iter = max(it.nkv0, it.nkv1);
        return it;
    };

    if (tid == 0) {
        *abort_flag = 0;
        mbar_init(q_full, 1);
        mbar_init(q_free, 1);
        mbar_init(k0_free, 1);
        for (int s = 0; s < KS; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1); }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&s_full[i], 1); mbar_init(&p_half[2 * i], 4); mbar_init(&p_half[2 * i + 1], 4);
            mbar_init(&o_full[i], 1); mbar_init(&o_free[i], 4);
        }
        mbar_init(stage_free, 1);
        item_ring_init(ring, 9);                 // readers: the MMA warp and the eight softmax warps
        fence_mbar_init();
    }
    if (warp == 8) { tmem_alloc(tmem_slot, TR::TM_COLS); tmem_relinquish(); }
    if (warp == 9 && lane == 0) {
        tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_k); tma_prefetch_desc(&tm_v); tma_prefetch_desc(&tm_o);
        if constexpr (TR::SPLIT) { tma_prefetch_desc(&tm_q_lo); tma_prefetch_desc(&tm_k_lo); tma_prefetch_desc(&tm_v_lo); }
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    if (warp >= 8) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
    }
    if (warp == 9) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            uint32_t G = 0;                               // load groups issued so far (= K tiles = V tiles loaded before this item)
            int n = 0;
            for (int idx = blockIdx.x; idx < pp.n_items; ++n) {
                if (*abort_flag != 0) break;
                const Item it = decode(idx);
                // draw the next item now; the value is needed (and published to the other roles) only after this item's first loads
                const int drawn = atomicAdd(pp.next_item, 1);
                if (n > 0) mbar_wait(q_free, (n - 1) & 1, ab, 12);
                const int q_tiles = (it.nkv1 > 0) ? 2 : 1;
                mbar_arrive_expect_tx(q_full, (q_tiles + 1) * TR::TILE_BYTES);
                // panel p of a tile: columns 64p.. of a bf16 operand, or (fp32 I/O) the hi / lo half of the bf16 pair
                auto col = [](int p) { return TR::SPLIT ? 0 : p * 64; };
                for (int p = 0; p < TR::NP; ++p) tma_load_4d(sQ + p * TR::PANEL_BYTES, (TR::SPLIT && p) ? &tm_q_lo : &tm_q, q_full, col(p), it.m0 * BM, it.hd, it.bt);
                if (q_tiles == 2)
                    for (int p = 0; p < TR::NP; ++p)
                        tma_load_4d(sQ + TR::TILE_BYTES + p * TR::PANEL_BYTES, (TR::SPLIT && p) ? &tm_q_lo : &tm_q, q_full, col(p), it.m1 * BM, it.hd, it.bt);
                for (int p = 0; p < TR::NP; ++p)
                    tma_load_4d(sK + (G % KS) * TR::TILE_BYTES + p * TR::PANEL_BYTES, (TR::SPLIT && p) ? &tm_k_lo : &tm_k, q_full, col(p), 0, it.hd, it.bt);
                idx = static_cast<int>(gridDim.x) + drawn;
                item_ring_publish(ring, n, idx, ab);
                for (int j = 0; j < it.n_iter; ++j, ++G) {
                    const int s = G % KS;
                    const bool has_k = (j + 1) < it.n_iter;
                    mbar_wait(&kv_empty[s], ((G / KS) & 1) ^ 1, ab, 10);
                    if (j == KS - 1) mbar_wait(k0_free, n & 1, ab, 11);         // K_KS reuses the slot of K_0
                    mbar_arrive_expect_tx(&kv_full[s], (has_k ? 2 : 1) * TR::TILE_BYTES);
                    if (has_k)
                        for (int p = 0; p < TR::NP; ++p)
                            tma_load_4d(sK + ((G + 1) % KS) * TR::TILE_BYTES + p * TR::PANEL_BYTES, (TR::SPLIT && p) ? &tm_k_lo : &tm_k, &kv_full[s], col(p),
                                        (j + 1) * BN, it.hd, it.bt);
                    for (int p = 0; p < TR::NP; ++p)
                        tma_load_4d(sV + s * TR::TILE_BYTES + p * TR::PANEL_BYTES, (TR::SPLIT && p) ? &tm_v_lo : &tm_v, &kv_full[s], col(p), j * BN, it.hd, it.bt);
                }
            }
        }
    } else if (warp == 8) {
        // ------------------------------ MMA issuer (converged warp, one elected lane issues) ------------------------------
        const bool leader = elect_one_lane();
        const uint32_t k_lo0 = sdesc_lo(smem_u32(sK), 16), v_lo0 = sdesc_lo(smem_u32(sV), TR::PANEL_BYTES);
        const uint32_t q_lo[2] = {sdesc_lo(smem_u32(sQ), 16), sdesc_lo(smem_u32(sQ + TR::TILE_BYTES), 16)};
        constexpr uint32_t kStage = TR::TILE_BYTES >> 4;
        uint32_t G = 0;
        uint32_t pc[2] = {0, 0};          // P tiles consumed so far per query tile (phase of p_half)
        uint32_t oc[2] = {0, 0};          // items in which query tile i was valid (phase of o_free)
        int n = 0;
        for (int idx = blockIdx.x; idx < pp.n_items; idx = item_ring_next(ring, n++, ab, leader)) {
            if (*abort_flag != 0) break;
            const Item it = decode(idx);
            const int nkv[2] = {it.nkv0, it.nkv1};
            mbar_wait(q_full, n & 1, ab, 20);
            tc_fence_after_sync();
#pragma unroll
            for (int i = 0; i < 2; ++i)
                if (nkv[i] > 0) {
                    fwd_issue_s<TR>(tmem + (i ? TR::TM_S1 : TR::TM_S0), q_lo[i], k_lo0 + (G % KS) * kStage, leader);
                    if (leader) umma_commit(&s_full[i]);
                }
            if (leader) umma_commit(k0_free);
            if (it.n_iter == 1 && leader) umma_commit(q_free);
            for (int j = 0; j < it.n_iter; ++j, ++G) {
                const int sv = G % KS;
                const uint32_t v_lo = v_lo0 + sv * kStage, k_next_lo = k_lo0 + ((G + 1) % KS) * kStage;
                mbar_wait(&kv_full[sv], (G / KS) & 1, ab, 22);
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    if (j < nkv[i]) {
                        const uint32_t tm_s = tmem + (i ? TR::TM_S1 : TR::TM_S0), tm_o = tmem + (i ? TR::TM_O1 : TR::TM_O0);
                        // the first P.V of an item overwrites O_i: the previous item's epilogue must have read it
                        if (j == 0 && oc[i] > 0) mbar_wait(&o_free[i], (oc[i] - 1) & 1, ab, 26);
                        mbar_wait(&p_half[2 * i], pc[i] & 1, ab, 24);
                        tc_fence_after_sync();
                        if constexpr (!TR::SPLIT) {
                            fwd_issue_pv_part<TR, 0, TR::PV_KSTEPS / 2>(tm_o, tm_s, v_lo, j == 0, leader);
                            mbar_wait(&p_half[2 * i + 1], pc[i] & 1, ab, 25);
                            tc_fence_after_sync();
                            fwd_issue_pv_part<TR, TR::PV_KSTEPS / 2, TR::PV_KSTEPS>(tm_o, tm_s, v_lo, j == 0, leader);
                        } else {
                            mbar_wait(&p_half[2 * i + 1], pc[i] & 1, ab, 25);
                            tc_fence_after_sync();
                            fwd_issue_pv<TR>(tm_o, tm_s, v_lo, j == 0, leader);
                        }
                        ++pc[i];
                        if (j + 1 < nkv[i]) {
                            fwd_issue_s<TR>(tm_s, q_lo[i], k_next_lo, leader);
                            if (leader) umma_commit(&s_full[i]);
                        } else {
                            if (leader) umma_commit(&o_full[i]);           // last key tile of this query tile: O_i is final
                            ++oc[i];
                        }
                    }
                }
                if (leader) umma_commit(&kv_empty[sv]);
                // the item's last S MMAs were issued in iteration n_iter - 2: Q and the K slots are free once they complete
                if (j == it.n_iter - 2 && leader) umma_commit(q_free);
            }
        }
    } else if (warp < 8) {
        // ------------------------------ softmax groups ------------------------------
        asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
        const int i = warp >> 2;                 // query tile handled by this group
        const int t = tid & 127;                 // row inside the tile
        const int wq = warp & 3;                 // TMEM lane quarter
        const uint32_t lane_base = static_cast<uint32_t>(wq * 32) << 16;
        const uint32_t tm_s = tmem + (i ? TR::TM_S1 : TR::TM_S0) + lane_base;
        const uint32_t tm_oo = tmem + (i ? TR::TM_O1 : TR::TM_O0) + lane_base;
        const float c = prm.scale_log2;
        uint32_t sc = 0;                         // S tiles consumed so far (phase of s_full)
        uint32_t oc = 0;                         // items in which this query tile was valid (phase of o_full)
        int n = 0;
        for (int idx = blockIdx.x; idx < pp.n_items; idx = item_ring_next(ring, n++, ab, lane == 0)) {
            if (*abort_flag != 0) break;
            const Item it = decode(idx);
            const int nkv = i ? it.nkv1 : it.nkv0;
            const int m_tile = i ? it.m1 : it.m0;
            const int row_g = m_tile * BM + t;
            float m_used = 0.f, l = 0.f;

            for (int j = 0; j < nkv; ++j, ++sc) {
                mbar_wait(&s_full[i], sc & 1, ab, 30);
                tc_fence_after_sync();
                float s[BN];
#pragma unroll
                for (int cc = 0; cc < BN; cc += 32) {
                    uint32_t r[32];
                    tmem_ld_x32(tm_s + cc, r);
#pragma unroll
                    for (int e = 0; e < 32; ++e) s[cc + e] = __uint_as_float(r[e]);
                }
                tmem_wait_ld();
                // masking: causal on the diagonal tile; keys past T on the last tile
                const int col0 = j * BN;
                const bool diag = prm.causal && (j == m_tile);
                const bool tail = (col0 + BN > T);
                if (diag || tail) {
                    const int limit = diag ? min(row_g, T - 1) : (T - 1);   // last visible key
#pragma unroll
                    for (int e = 0; e < BN; ++e)
                        if (col0 + e > limit) s[e] = -INFINITY;
                }
                // row maximum: eight independent chains (a single 127-deep chain would expose its full latency)
                float mx8[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) mx8[e] = s[e];
#pragma unroll
                for (int u = 0; u < 8; ++u) mx8[u] = fmaxf(mx8[u], s[8 + u]);
#pragma unroll
                for (int e = 16; e < BN; e += 16)
#pragma unroll
                    for (int u = 0; u < 8; ++u) mx8[u] = fmax3(mx8[u], s[e + u], s[e + 8 + u]);
                const float mx = fmax3(fmax3(mx8[0], mx8[1], mx8[2]), fmax3(mx8[3], mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7]));
                float mx_s = mx * c;
                if (mx == -INFINITY) mx_s = m_used;                    // fully masked row in this tile
                if (j == 0) {
                    m_used = (mx == -INFINITY) ? 0.f : mx_s;
                } else {
                    const bool need = mx_s > m_used + kRescaleLog2;
                    if (__any_sync(0xffffffffu, need)) {
                        // P.V_{j-1} has completed: this iteration's S commit was issued after it
                        const float alpha = need ? fast_exp2(m_used - mx_s) : 1.f;
                        if (need) { m_used = mx_s; l *= alpha; }
#pragma unroll
                        for (int cc = 0; cc < D; cc += 32) {
                            uint32_t r[32];
                            tmem_ld_x32(tm_oo + cc, r);
                            tmem_wait_ld();
#pragma unroll
                            for (int e = 0; e < 32; ++e) r[e] = __float_as_uint(__uint_as_float(r[e]) * alpha);
                            tmem_st_x32(tm_oo + cc, r);
                        }
                        tmem_wait_st();
                    }
                }
                // P = exp2(s * c - m): packed fp32x2 FMA, row sum in four independent packed accumulators
                const uint64_t c2 = pack_f32x2(c, c), nm2 = pack_f32x2(-m_used, -m_used);
                uint64_t acc2[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
                for (int cc = 0; cc < BN; cc += 32) {
                    uint32_t pk[16], pl[16];
#pragma unroll
                    for (int e = 0; e < 32; e += 2) {
                        float x0, x1;
                        unpack_f32x2(ffma2(pack_f32x2(s[cc + e], s[cc + e + 1]), c2, nm2), x0, x1);
                        const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
                        acc2[(e >> 1) & 3] = fadd2(acc2[(e >> 1) & 3], pack_f32x2(p0, p1));
                        const uint32_t hi = pack_bf16x2(p0, p1);
                        pk[e >> 1] = hi;
                        if constexpr (TR::SPLIT)
                            pl[e >> 1] = pack_bf16x2(p0 - __uint_as_float(hi << 16), p1 - __uint_as_float(hi & 0xffff0000u));
                    }
                    if (cc == BN / 2) {
                        // columns 0-63 were stored a chunk ago: publish them (the wait returns at once)
                        tmem_wait_st();
                        tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&p_half[2 * i]);
                    }
                    tmem_st_x16(tm_s + (cc >> 1), pk);
                    if constexpr (TR::SPLIT) tmem_st_x16(tm_s + 64 + (cc >> 1), pl);
                }
                {
                    float a0, a1;
                    unpack_f32x2(fadd2(fadd2(acc2[0], acc2[1]), fadd2(acc2[2], acc2[3])), a0, a1);
                    l += a0 + a1;
                }
                tmem_wait_st();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(&p_half[2 * i + 1]);
            }

            // ---- epilogue of this query tile; the staging tile is used by tile 0 and tile 1 of every item in turn ----
            const uint32_t use = 2u * static_cast<uint32_t>(n) + static_cast<uint32_t>(i);
            if (nkv > 0) {
                mbar_wait(&o_full[i], oc & 1, ab, 32);
                ++oc;
                tc_fence_after_sync();
                const float inv_l = 1.f / l;
                if (use > 0) mbar_wait(stage_free, (use - 1) & 1, ab, 33);
#pragma unroll
                for (int cc = 0; cc < D; cc += 32) {
                    uint32_t r[32];
                    tmem_ld_x32(tm_oo + cc, r);
                    tmem_wait_ld();
                    if (cc + 32 == D) {
                        // O_i is in registers: the next item's first P.V may overwrite it
                        tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&o_free[i]);
                    }
                    if constexpr (!TR::SPLIT) {
                        // 32 columns = 64 bytes = 4 chunks of 16 B inside panel cc/64
                        const int panel = cc / 64, chunk0 = (cc % 64) / 8;
#pragma unroll
                        for (int q4 = 0; q4 < 4; ++q4) {
                            uint4 v;
                            v.x = pack_bf16x2(__uint_as_float(r[q4 * 8 + 0]) * inv_l, __uint_as_float(r[q4 * 8 + 1]) * inv_l);
                            v.y = pack_bf16x2(__uint_as_float(r[q4 * 8 + 2]) * inv_l, __uint_as_float(r[q4 * 8 + 3]) * inv_l);
                            v.z = pack_bf16x2(__uint_as_float(r[q4 * 8 + 4]) * inv_l, __uint_as_float(r[q4 * 8 + 5]) * inv_l);
                            v.w = pack_bf16x2(__uint_as_float(r[q4 * 8 + 6]) * inv_l, __uint_as_float(r[q4 * 8 + 7]) * inv_l);
                            st_shared_sw128(sO + panel * TR::PANEL_BYTES, t, chunk0 + q4, v);
                        }
                    } else {
                        // 32 fp32 columns = one 128-byte panel row = 8 chunks of 16 B
                        const int panel = cc / 32;
#pragma unroll
                        for (int q4 = 0; q4 < 8; ++q4) {
                            uint4 v;
                            v.x = __float_as_uint(__uint_as_float(r[q4 * 4 + 0]) * inv_l);
                            v.y = __float_as_uint(__uint_as_float(r[q4 * 4 + 1]) * inv_l);
                            v.z = __float_as_uint(__uint_as_float(r[q4 * 4 + 2]) * inv_l);
                            v.w = __float_as_uint(__uint_as_float(r[q4 * 4 + 3]) * inv_l);
                            st_shared_sw128(sO + panel * TR::PANEL_BYTES, t, q4, v);
                        }
                    }
                }
                if (row_g < T) prm.lse[static_cast<size_t>(it.bh) * T + row_g] = (m_used + log2f(l)) * 0.6931471805599453f;
                fence_proxy_async_smem();
                asm volatile("bar.sync %0, 128;" ::"r"(1 + i) : "memory");
                if (t == 0) {
                    for (int p = 0; p < TR::OUT_PANELS; ++p)
                        tma_store_4d(&tm_o, sO + p * TR::PANEL_BYTES, p * TR::OUT_PANEL_ELEMS, m_tile * BM, it.hd, it.bt);
                    tma_store_commit();
                    tma_store_wait_read_all();
                    mbar_arrive(stage_free);
                }
            } else if (t == 0) {
                // a query tile past T: keep the staging tile's turn order
                if (use > 0) mbar_wait(stage_free, (use - 1) & 1, ab, 34);
                mbar_arrive(stage_free);
            }
        }
    }

    // ------------------------------ tear-down ------------------------------
    tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag != 0) {
        // a wait gave up: give any TMA copy still in flight time to land before the CTA's shared memory is released
        for (int it = 0; it < 64; ++it) __nanosleep(1000);
    }
    if (warp == 8) tmem_dealloc(tmem, TR::TM_COLS);
}

}  // namespace ib200
