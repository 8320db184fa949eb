// Causal flash-attention forward for sm_100a.
//
// Replaces the reference's composed forward
//   matmul(q,kt) -> * scale -> triu/masked_fill(-1e9) -> Softmax -> matmul(attn,v)
// (InfernoApp/main.cpp:737-754; ops in src/inferno/core/ops.cpp:437-735, 204-270,
// 1235-1289, 1355-1398; src/inferno/functional/softmax.cpp:22-79) with one kernel
// that never materialises the [T,T] score matrix and saves the per-row
// log-sum-exp for the backward pass.
//
// One CTA owns two adjacent 128-row query tiles of one (batch, head) and walks the
// key/value tiles up to the diagonal:
//   warps 10-11 idle (they only donate registers)
//   warp 9      TMA producer: the Q tiles and K_0 once, then one load group {K_{j+1}, V_j}
//               per iteration (exactly what iteration j of the MMA warp consumes)
//   warp 8      MMA issuer: the warp stays converged and one elected lane issues
//               S_i = Q_i K_j^T (smem x smem -> TMEM) and O_i += P_i V_j (P read from
//               TMEM, V from smem, MN-major)
//   warps 0-3   softmax for query tile 0 (one thread per row, no shuffles needed:
//               the 32x32b TMEM load gives each thread a whole row)
//   warps 4-7   softmax for query tile 1
// While one softmax group exponentiates, the tensor core works for the other.
// P overwrites S in place in TMEM and is published to the MMA warp in two halves of 64
// keys.  O stays in TMEM for the whole walk; it is rescaled only when a row maximum
// grows by more than 2^kRescaleLog2 ("lazy" rescale), which the final division by the
// row sum makes exact.
#pragma once

#include "sm100_ptx.cuh"

namespace ib200 {

// SPLIT = false: bf16 operands and output, head dim D (64 or 128).
// SPLIT = true : fp32 I/O for D = 64.  Every fp32 operand x is carried as two bf16 tensors,
//   x_hi = bf16(x) and x_lo = bf16(x - x_hi); a product a*b is evaluated as
//   a_hi*b_hi + a_lo*b_hi + a_hi*b_lo on the bf16 tensor pipe with fp32 accumulation
//   (relative error ~2^-16 per product, below a single TF32 pass at 2^-11).  The hi and
//   lo tiles take the place of the two 64-column panels of a D = 128 tile, so the shared
//   memory and TMEM budgets are those of the bf16 D = 128 kernel.
template <int D_, bool SPLIT_>
struct FwdTraits {
    static constexpr int D = D_;
    static constexpr bool SPLIT = SPLIT_;
    static_assert(!SPLIT || D == 64, "split-bf16 mode is built for head dim 64");
    static constexpr int BM = 128, BN = 128;                // query / key tile rows
    static constexpr int NP = SPLIT ? 2 : D / 64;           // 128-byte panels per operand tile (hi/lo or column halves)
    static constexpr int PANEL_BYTES = 128 * 128;           // [128 rows x 128 B]
    static constexpr int TILE_BYTES = NP * PANEL_BYTES;
    static constexpr int NTERMS = SPLIT ? 3 : 1;
    static constexpr int PV_KSTEPS = BN / 16;               // k-steps of P V (16 keys each)
    static constexpr int KV_STAGES = (TILE_BYTES <= 16384) ? 4 : 2;
    static constexpr uint32_t IDESC_S = make_idesc(kFmtBF16, BM, BN, kMajorK, kMajorK);
    static constexpr uint32_t IDESC_PV = make_idesc(kFmtBF16, BM, D, kMajorK, kMajorMN);
    // TMEM columns: S0, S1 (128 each), O0, O1 (D each, padded to 128)
    static constexpr uint32_t TM_S0 = 0, TM_S1 = 128, TM_O0 = 256, TM_O1 = 384, TM_COLS = 512;
    static constexpr int OUT_PANELS = SPLIT ? 2 : D / 64;   // output staging panels ([128 x 128 B] each)
    static constexpr int OUT_PANEL_ELEMS = SPLIT ? 32 : 64;
    static constexpr int SMEM_TILES = 2 + 2 * KV_STAGES;
    static constexpr int SMEM_BYTES = SMEM_TILES * TILE_BYTES + 1024 /*align slack*/ + 512 /*barriers*/;
    static constexpr int THREADS = 384;                      // 3 warpgroups: softmax 0, softmax 1, {MMA, TMA, 2 idle}
};

struct FwdParams {
    float* lse;            // [BH, T] natural-log units, scale included
    int* status;           // device status word (0 = ok)
    int T, BH, H;          // H: heads per batch entry (the tensor maps are 4-D: column, token, head, batch)
    int causal;
    float scale_log2;      // scale * log2(e)
};

constexpr float kRescaleLog2 = 8.0f;

// Operand panel used by term t of a split product: a_hi*b_hi, a_lo*b_hi, a_hi*b_lo.
__device__ __forceinline__ constexpr int split_a(int t) { return t == 1 ? 1 : 0; }
__device__ __forceinline__ constexpr int split_b(int t) { return t == 2 ? 1 : 0; }

// The issue helpers take descriptor LOW WORDS (sdesc_lo) so that each MMA costs one 32-bit add per operand.
template <class TR>
__device__ __forceinline__ void fwd_issue_s(uint32_t tmem_s, uint32_t q_lo, uint32_t k_lo, bool leader) {
    if constexpr (!TR::SPLIT) {
#pragma unroll
        for (int k = 0; k < TR::D / 16; ++k) {
            const uint32_t off = ((k / 4) * TR::PANEL_BYTES + (k % 4) * 32) >> 4;
            if (leader) umma_ss_f16(tmem_s, sdesc_join(q_lo + off), sdesc_join(k_lo + off), TR::IDESC_S, k > 0);
        }
    } else {
#pragma unroll
        for (int t = 0; t < 3; ++t)
#pragma unroll
            for (int k = 0; k < 4; ++k)
                if (leader) umma_ss_f16(tmem_s, sdesc_join(q_lo + ((split_a(t) * TR::PANEL_BYTES + k * 32) >> 4)),
                            sdesc_join(k_lo + ((split_b(t) * TR::PANEL_BYTES + k * 32) >> 4)), TR::IDESC_S, (t | k) != 0);
    }
}

// v_lo_mn: low word of V's MN-major view (lbo = panel stride).
template <class TR, int K0, int K1>
__device__ __forceinline__ void fwd_issue_pv_part(uint32_t tmem_o, uint32_t tmem_p, uint32_t v_lo_mn, bool first_tile, bool leader) {
    static_assert(!TR::SPLIT, "bf16 mode only");
#pragma unroll
    for (int k = K0; k < K1; ++k)
        if (leader) umma_ts_f16(tmem_o, tmem_p + k * 8, sdesc_join(v_lo_mn + ((k * 2048) >> 4)), TR::IDESC_PV, (!first_tile || k > 0) ? 1u : 0u);
}

template <class TR>
__device__ __forceinline__ void fwd_issue_pv(uint32_t tmem_o, uint32_t tmem_p, uint32_t v_lo_mn, bool first_tile, bool leader) {
    if constexpr (!TR::SPLIT) {
#pragma unroll
        for (int k = 0; k < TR::PV_KSTEPS; ++k)
            if (leader) umma_ts_f16(tmem_o, tmem_p + k * 8, sdesc_join(v_lo_mn + ((k * 2048) >> 4)), TR::IDESC_PV, (!first_tile || k > 0) ? 1u : 0u);
    } else {
        // P_hi in columns 0-63, P_lo in columns 64-127 of the S region; V_hi / V_lo are the two panels
#pragma unroll
        for (int t = 0; t < 3; ++t)
#pragma unroll
            for (int k = 0; k < TR::PV_KSTEPS; ++k)
                if (leader) umma_ts_f16(tmem_o, tmem_p + split_a(t) * 64 + k * 8, sdesc_join(v_lo_mn + ((split_b(t) * TR::PANEL_BYTES + k * 2048) >> 4)),
                            TR::IDESC_PV, (!first_tile || (t | k) != 0) ? 1u : 0u);
    }
}

template <class TR>
__global__ void __launch_bounds__(TR::THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_q_lo,
                const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_k_lo,
                const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_v_lo,
                const __grid_constant__ CUtensorMap tm_o, FwdParams prm) {
    constexpr int D = TR::D, BM = TR::BM, BN = TR::BN, KS = TR::KV_STAGES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint8_t* sQ = smem;                                   // 2 tiles (reused as O staging)
    uint8_t* sK = sQ + 2 * TR::TILE_BYTES;                // KS tiles
    uint8_t* sV = sK + KS * TR::TILE_BYTES;               // KS tiles
    uint64_t* bars = reinterpret_cast<uint64_t*>(sV + KS * TR::TILE_BYTES);
    uint64_t* q_full = bars;                // [1]   query tiles + K_0
    uint64_t* k0_free = bars + 1;           // [1]   the first S MMAs have read K_0
    uint64_t* kv_full = bars + 2;           // [KS]  load group j: K_{j+1} and V_j
    uint64_t* kv_empty = kv_full + KS;      // [KS]
    uint64_t* s_full = kv_empty + KS;       // [2]   S_i is in TMEM (and every MMA issued before it has completed)
    uint64_t* p_half = s_full + 2;          // [2][2]  P columns 0-63 / 64-127 of tile i are in TMEM
    uint64_t* o_full = p_half + 4;          // [2]   after the last P.V of tile i
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_full + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int T = prm.T;
    const int bh = blockIdx.y;
    const int hd = bh % prm.H, bt = bh / prm.H;            // head and batch coordinates
    const int pair = (gridDim.x - 1) - blockIdx.x;          // heaviest (longest walk) first
    const int m_tile[2] = {2 * pair, 2 * pair + 1};
    const int n_kv_total = (T + BN - 1) / BN;
    int n_kv[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const bool valid = m_tile[i] * BM < T;
        n_kv[i] = !valid ? 0 : (prm.causal ? min(m_tile[i] + 1, n_kv_total) : n_kv_total);
    }
    const int n_iter = max(n_kv[0], n_kv[1]);
    AbortCtx ab{abort_flag, prm.status};

    if (tid == 0) {
        *abort_flag = 0;
        mbar_init(q_full, 1);
        mbar_init(k0_free, 1);
        for (int s = 0; s < KS; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(&s_full[i], 1); mbar_init(&p_half[2 * i], 4); mbar_init(&p_half[2 * i + 1], 4); mbar_init(&o_full[i], 1); }
        fence_mbar_init();
    }
    if (warp == 8) { tmem_alloc(tmem_slot, TR::TM_COLS); tmem_relinquish(); }
    if (warp == 9 && lane == 0) { tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_k); tma_prefetch_desc(&tm_v); tma_prefetch_desc(&tm_o);
        if constexpr (TR::SPLIT) { tma_prefetch_desc(&tm_q_lo); tma_prefetch_desc(&tm_k_lo); tma_prefetch_desc(&tm_v_lo); } }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    // Register rebalancing between warpgroups (the launch gives every thread 168).
    if (warp >= 8) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
    }
    if (warp == 9) {
        // ------------------------------ TMA producer ------------------------------
        // Load group j = {K_{j+1}, V_j}: exactly what iteration j of the MMA issuer consumes (P.V_j, then S = Q K_{j+1}^T),
        // so a group needs one full and one empty barrier.  K_j lives in K slot j % KS, V_j in V slot j % KS; K_0 comes
        // with the query tiles.
        if (lane == 0) {
            const int q_tiles = (n_kv[1] > 0) ? 2 : 1;
            mbar_arrive_expect_tx(q_full, (q_tiles + 1) * TR::TILE_BYTES);
            for (int i = 0; i < q_tiles; ++i)
                for (int p = 0; p < TR::NP; ++p)
                    tma_load_4d(sQ + i * TR::TILE_BYTES + p * TR::PANEL_BYTES, (TR::SPLIT && p) ? &tm_q_lo : &tm_q, q_full, TR::SPLIT ? 0 : p * 64, m_tile[i] * BM, hd, bt);
            for (int p = 0; p < TR::NP; ++p)
                tma_load_4d(sK + p * TR::PANEL_BYTES, (TR::SPLIT && p) ? &tm_k_lo : &tm_k, q_full, TR::SPLIT ? 0 : p * 64, 0, hd, bt);
            for (int j = 0; j < n_iter; ++j) {
                const int s = j % KS;
                const bool has_k = (j + 1) < n_iter;
                mbar_wait(&kv_empty[s], ((j / KS) & 1) ^ 1, ab, 10);
                if (j == KS - 1) mbar_wait(k0_free, 0, ab, 11);            // K_KS reuses the slot of K_0
                mbar_arrive_expect_tx(&kv_full[s], (has_k ? 2 : 1) * TR::TILE_BYTES);
                if (has_k)
                    for (int p = 0; p < TR::NP; ++p)
                        tma_load_4d(sK + ((j + 1) % KS) * TR::TILE_BYTES + p * TR::PANEL_BYTES, (TR::SPLIT && p) ? &tm_k_lo : &tm_k, &kv_full[s],
                                    TR::SPLIT ? 0 : p * 64, (j + 1) * BN, hd, bt);
                for (int p = 0; p < TR::NP; ++p)
                    tma_load_4d(sV + s * TR::TILE_BYTES + p * TR::PANEL_BYTES, (TR::SPLIT && p) ? &tm_v_lo : &tm_v, &kv_full[s], TR::SPLIT ? 0 : p * 64, j * BN, hd, bt);
            }
        }
    } else if (warp == 8) {
        // ------------------------------ MMA issuer ------------------------------
        // The whole warp walks the loop converged and only the MMA / commit instructions are predicated on one elected
        // lane (a converged warp issues an MMA every ~39 cycles and commits for free; a lone lane in a divergent branch
        // pays ~44 per MMA and ~44 more per commit).  Waits and commits cost tensor-pipe time (its queue is about one MMA
        // deep), so there are as few as the hazards allow: per iteration one wait for the K/V group, two per query tile
        // for the halves of P, one commit per tile (S ready; since a commit covers everything issued before it, it also
        // tells the softmax that the previous P.V has completed) and one commit that frees the K/V group.
        if (n_iter > 0) {
            const bool leader = elect_one_lane();
            const uint32_t k_lo0 = sdesc_lo(smem_u32(sK), 16), v_lo0 = sdesc_lo(smem_u32(sV), TR::PANEL_BYTES);
            constexpr uint32_t kStage = TR::TILE_BYTES >> 4;
            mbar_wait(q_full, 0, ab, 20);
            tc_fence_after_sync();
#pragma unroll
            for (int i = 0; i < 2; ++i)
                if (n_kv[i] > 0) {
                    fwd_issue_s<TR>(tmem + (i ? TR::TM_S1 : TR::TM_S0), sdesc_lo(smem_u32(sQ + i * TR::TILE_BYTES), 16), k_lo0, leader);
                    if (leader) umma_commit(&s_full[i]);
                }
            if (leader) umma_commit(k0_free);
            for (int j = 0; j < n_iter; ++j) {
                const int sv = j % KS;
                const uint32_t v_lo = v_lo0 + sv * kStage, k_next_lo = k_lo0 + ((j + 1) % KS) * kStage;
                mbar_wait(&kv_full[sv], (j / KS) & 1, ab, 22);
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    if (j < n_kv[i]) {
                        const uint32_t tm_s = tmem + (i ? TR::TM_S1 : TR::TM_S0), tm_o = tmem + (i ? TR::TM_O1 : TR::TM_O0);
                        // P arrives in two halves of 64 key columns: the first k-steps of P.V run under the second half's exponentials
                        mbar_wait(&p_half[2 * i], j & 1, ab, 24);
                        tc_fence_after_sync();
                        if constexpr (!TR::SPLIT) {
                            fwd_issue_pv_part<TR, 0, TR::PV_KSTEPS / 2>(tm_o, tm_s, v_lo, j == 0, leader);
                            mbar_wait(&p_half[2 * i + 1], j & 1, ab, 25);
                            tc_fence_after_sync();
                            fwd_issue_pv_part<TR, TR::PV_KSTEPS / 2, TR::PV_KSTEPS>(tm_o, tm_s, v_lo, j == 0, leader);
                        } else {
                            mbar_wait(&p_half[2 * i + 1], j & 1, ab, 25);
                            tc_fence_after_sync();
                            fwd_issue_pv<TR>(tm_o, tm_s, v_lo, j == 0, leader);
                        }
                        if (j + 1 < n_kv[i]) {
                            fwd_issue_s<TR>(tm_s, sdesc_lo(smem_u32(sQ + i * TR::TILE_BYTES), 16), k_next_lo, leader);
                            if (leader) umma_commit(&s_full[i]);
                        } else {
                            if (leader) umma_commit(&o_full[i]);           // last key tile of this query tile: O_i is final
                        }
                    }
                }
                if (leader) umma_commit(&kv_empty[sv]);
            }
        }
    } else if (warp < 8) {
        // ------------------------------ softmax groups ------------------------------
        asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
        const int i = warp >> 2;                 // query tile handled by this group
        const int t = tid & 127;                 // row inside the tile
        const int wq = warp & 3;                 // TMEM lane quarter
        const int nkv = n_kv[i];
        const int row_g = m_tile[i] * BM + t;
        const uint32_t lane_base = static_cast<uint32_t>(wq * 32) << 16;
        const uint32_t tm_s = tmem + (i ? TR::TM_S1 : TR::TM_S0) + lane_base;
        const uint32_t tm_oo = tmem + (i ? TR::TM_O1 : TR::TM_O0) + lane_base;
        const float c = prm.scale_log2;
        float m_used = 0.f, l = 0.f;

        for (int j = 0; j < nkv; ++j) {
            mbar_wait(&s_full[i], j & 1, ab, 30);
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
            const bool diag = prm.causal && (j == m_tile[i]);
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
            for (int e = 8; e < BN; e += 8)
#pragma unroll
                for (int u = 0; u < 8; ++u) mx8[u] = fmaxf(mx8[u], s[e + u]);
            const float mx = fmaxf(fmaxf(fmaxf(mx8[0], mx8[1]), fmaxf(mx8[2], mx8[3])), fmaxf(fmaxf(mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7])));
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
            float lsum;
            {
                float a0, a1;
                unpack_f32x2(fadd2(fadd2(acc2[0], acc2[1]), fadd2(acc2[2], acc2[3])), a0, a1);
                lsum = a0 + a1;
            }
            l += lsum;
            tmem_wait_st();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_half[2 * i + 1]);
        }

        if (nkv > 0) {
            mbar_wait(&o_full[i], 0, ab, 32);
            tc_fence_after_sync();
            const float inv_l = 1.f / l;
            uint8_t* stage = sQ + i * TR::TILE_BYTES;     // Q_i is dead once its last S MMA has completed
#pragma unroll
            for (int cc = 0; cc < D; cc += 32) {
                uint32_t r[32];
                tmem_ld_x32(tm_oo + cc, r);
                tmem_wait_ld();
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
                        st_shared_sw128(stage + panel * TR::PANEL_BYTES, t, chunk0 + q4, v);
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
                        st_shared_sw128(stage + panel * TR::PANEL_BYTES, t, q4, v);
                    }
                }
            }
            if (row_g < T) prm.lse[static_cast<size_t>(bh) * T + row_g] = (m_used + log2f(l)) * 0.6931471805599453f;
            fence_proxy_async_smem();
            asm volatile("bar.sync %0, 128;" ::"r"(1 + i) : "memory");
            if (t == 0) {
                for (int p = 0; p < TR::OUT_PANELS; ++p)
                    tma_store_4d(&tm_o, stage + p * TR::PANEL_BYTES, p * TR::OUT_PANEL_ELEMS, m_tile[i] * BM, hd, bt);
                tma_store_commit();
                tma_store_wait_read_all();     // the CTA may leave once its shared memory has been read; the writes complete on their own
            }
        }
    }

    // ------------------------------ tear-down ------------------------------
    tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag != 0) {
        // a wait gave up: give any TMA copy still in flight time to land before the CTA's
        // shared memory is released
        for (int it = 0; it < 64; ++it) __nanosleep(1000);
    }
    if (warp == 8) tmem_dealloc(tmem, TR::TM_COLS);
}

}  // namespace ib200
