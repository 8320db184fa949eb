// Causal flash-attention backward for sm_100a.
//
// Replaces the reference's backward node chain for the attention sub-graph
//   MMBackward(attn, v)   dP = dO V^T, dV = P^T dO      src/inferno/gradfn/mmbackward.cpp:36-98
//   SoftmaxBackward       dS = P * (dP - rowsum(dP*P))  src/inferno/gradfn/softmaxbackward.cpp:36-128
//   (masked_fill has no backward node in the reference; dS is 0 where masked because P is 0)
//   MultiplyBackward      dS *= scale                   src/inferno/gradfn/multiplybackward.cpp:34-57
//   MMBackward(q, kt)     dQ = dS K, dK = dS^T Q        src/inferno/gradfn/mmbackward.cpp:36-98
// with a kernel that recomputes P from Q, K and the saved log-sum-exp instead of
// reading a stored [T,T] matrix, and takes rowsum(dP*P) as delta = rowsum(dO*O).
//
// One CTA owns one 128-row key/value tile of one (batch, head) and walks the
// 64-row query blocks at or below the diagonal.  Everything is computed
// transposed (key index on the TMEM lanes) so that P^T and dS^T can feed the
// dV / dK MMAs straight from TMEM:
//   S^T  = K Q^T        smem x smem  -> TMEM ST[b]          (M=128 keys, N=64 queries)
//   dP^T = V dO^T       smem x smem  -> TMEM DP[b]
//   dV  += P^T dO       TMEM x smem (dO MN-major)   -> TMEM DV
//   dK  += dS^T Q       TMEM x smem (Q MN-major)    -> TMEM DK
//   dQ^T = K^T dS^T     smem (K MN-major) x smem (dS^T MN-major) -> TMEM DP[b]  (M=D, N=64)
// dQ^T is transposed through shared memory (lane = head-dim index, so a warp writes 32
// consecutive floats per store, conflict-free) and added to the fp32 scratch accumulator
// by a TMA reduction (cp.reduce.async.bulk.tensor .add), which keeps the adds off the
// load/store pipe the compute warps depend on.
//
// Software pipeline of the MMA issuer (block = one 64-row query block, b = block & 1):
//   prologue   S^T(0) dP^T(0) S^T(1) dP^T(1)
//   phase it   dQ^T(it) dK(it) dV(it) | S^T(it+2) dP^T(it+2)
// so the compute warps work on block it+1 while the tensor pipe runs phase it, and the
// drain of dQ^T(it) has three MMAs of slack before dP^T(it+2) reuses its TMEM buffer.
// P^T and dS^T (bf16) both live in the S^T buffer, so dQ^T may overwrite the dP^T
// buffer as soon as the compute warps have read it.
//
//   warps 0-7    compute: P^T = exp2(S^T c - lse), dS^T = P^T (dP^T - delta); each
//                thread owns one key row; warps 0-3 take query columns 0-31, 4-7 take 32-63
//   warps 8-11   drain dQ^T from TMEM to the global accumulator
//   warp 12      TMA producer (K, V once; Q, dO, lse, delta per query block)
//   warp 13      MMA issuer (converged warp, one elected lane issues)
#pragma once

#include "attn_aux.cuh"
#include "attn_fwd.cuh"
#include "sm100_ptx.cuh"

namespace ib200 {

// SPLIT = true is the fp32-I/O mode for D = 64 (see FwdTraits): every operand tile is a
// (hi, lo) bf16 pair occupying the two panels a D = 128 tile would, every product is three
// MMAs, and P^T / dS^T are split into hi and lo parts as well.
template <int D_, bool SPLIT_>
struct BwdTraits {
    static constexpr int D = D_;
    static constexpr bool SPLIT = SPLIT_;
    static_assert(!SPLIT || D == 64, "split-bf16 mode is built for head dim 64");
    static constexpr int BKV = 128, BQ = 64;
    static constexpr int NP = SPLIT ? 2 : D / 64;            // 128-byte panels per operand tile
    static constexpr int KV_PANEL = BKV * 128, KV_TILE = NP * KV_PANEL;
    static constexpr int Q_PANEL = BQ * 128, Q_TILE = NP * Q_PANEL;
    static constexpr int DS_PART = BKV * 128;                // [128 keys x 64 queries] bf16
    static constexpr int DS_TILE = (SPLIT ? 2 : 1) * DS_PART;
    static constexpr int NS = 3;                             // Q/dO ring depth
    static constexpr int NTERMS = SPLIT ? 3 : 1;
    static constexpr int OUT_TILE = SPLIT ? BKV * D * 4 : KV_TILE;   // dK / dV staging bytes
    static constexpr int OUT_PANELS = SPLIT ? 2 : D / 64;
    static constexpr int OUT_PANEL_ELEMS = SPLIT ? 32 : 64;
    static constexpr uint32_t IDESC_ST = make_idesc(kFmtBF16, BKV, BQ, kMajorK, kMajorK);
    static constexpr uint32_t IDESC_DKV = make_idesc(kFmtBF16, BKV, D, kMajorK, kMajorMN);
    static constexpr uint32_t IDESC_DQ = make_idesc(kFmtBF16, D, BQ, kMajorMN, kMajorMN);
    static constexpr uint32_t TM_ST = 0, TM_DP = 128, TM_DV = 256, TM_DK = 384, TM_COLS = 512;
    static constexpr int OFF_K = 0;
    static constexpr int OFF_V = OFF_K + KV_TILE;
    static constexpr int OFF_Q = OFF_V + KV_TILE;            // NS tiles; ring start, reused as dV/dK staging
    static constexpr int OFF_DO = OFF_Q + NS * Q_TILE;       // NS tiles
    static constexpr int OFF_DS = OFF_DO + NS * Q_TILE;      // one dS^T tile (hi + lo in split mode)
    static constexpr int OFF_DQ = OFF_DS + DS_TILE;          // dQ staging [64 queries x D] fp32, row-major, for the TMA reduction
    static constexpr int DQ_STAGE = BQ * D * 4;
    static constexpr int OFF_VEC = OFF_DQ + DQ_STAGE;     // NS x (lse[64], delta[64]) floats
    static constexpr int OFF_BAR = OFF_VEC + NS * 2 * BQ * 4;
    static constexpr int SMEM_BYTES = OFF_BAR + 512 + 1024;
    static constexpr int THREADS = 512;
    static_assert(2 * NS * Q_TILE >= 2 * OUT_TILE, "epilogue staging must fit in the Q/dO ring");
    static_assert(SMEM_BYTES <= 232448, "shared memory budget");
};

struct BwdParams {
    const float* nlse2;    // [BH, T_pad]  -lse * log2(e), 0 in the padding
    const float* ndelta;   // [BH, T_pad]  -rowsum(dO * O), 0 in the padding
    int T_pad;             // T rounded up to a multiple of 64
    int* status;
    int T, BH, H, causal;  // H: heads per batch entry (operand tensor maps are 4-D: column, token, head, batch)
    float scale, scale_log2;
};

// TMEM column of the packed bf16 pair that starts k-step ks (16 queries) of a P^T / dS^T operand.
// Each compute warpgroup owns 32 columns of a 64-column buffer (queries 0-31 -> columns 0-31,
// queries 32-63 -> columns 32-63) and writes only there; inside its 32 columns the first 16 hold
// "part 0" and the next 16 "part 1".  bf16 mode: S^T buffer = {P^T, dS^T}.  Split mode: S^T
// buffer = {P^T hi, P^T lo}, dP^T buffer = {dS^T hi, dS^T lo}.
__device__ __forceinline__ uint32_t bwd_pcol(int ks, int part = 0) { return static_cast<uint32_t>((ks >> 1) * 32 + (ks & 1) * 8 + part * 16); }

// The issue helpers take the LOW WORDS of the operands' shared-memory descriptors (sdesc_lo) so
// that every MMA costs one 32-bit add per operand in the issuing thread.

// acc[128 keys x 64 queries] = A B^T with A = K or V tile, B = Q or dO block, both K-major (S^T and dP^T).
template <class TR>
__device__ __forceinline__ void bwd_issue_kmajor(uint32_t tmem_acc, uint32_t a_lo, uint32_t b_lo, bool leader) {
    if constexpr (!TR::SPLIT) {
#pragma unroll
        for (int k = 0; k < TR::D / 16; ++k)
            if (leader) umma_ss_f16(tmem_acc, sdesc_join(a_lo + (((k / 4) * TR::KV_PANEL + (k % 4) * 32) >> 4)),
                        sdesc_join(b_lo + (((k / 4) * TR::Q_PANEL + (k % 4) * 32) >> 4)), TR::IDESC_ST, k > 0);
    } else {
#pragma unroll
        for (int t = 0; t < 3; ++t)
#pragma unroll
            for (int k = 0; k < 4; ++k)
                if (leader) umma_ss_f16(tmem_acc, sdesc_join(a_lo + ((split_a(t) * TR::KV_PANEL + k * 32) >> 4)),
                            sdesc_join(b_lo + ((split_b(t) * TR::Q_PANEL + k * 32) >> 4)), TR::IDESC_ST, (t | k) != 0);
    }
}

// acc[128 keys x D] += A B with A = P^T or dS^T in TMEM (64 queries), B = dO or Q block, MN-major (dV and dK).
template <class TR>
__device__ __forceinline__ void bwd_issue_acc(uint32_t tmem_acc, uint32_t tmem_a, int part, uint32_t b_lo_mn, bool accumulate, bool leader) {
    if constexpr (!TR::SPLIT) {
#pragma unroll
        for (int ks = 0; ks < TR::BQ / 16; ++ks)
            if (leader) umma_ts_f16(tmem_acc, tmem_a + bwd_pcol(ks, part), sdesc_join(b_lo_mn + ((ks * 2048) >> 4)), TR::IDESC_DKV,
                        (accumulate || ks > 0) ? 1u : 0u);
    } else {
#pragma unroll
        for (int t = 0; t < 3; ++t)
#pragma unroll
            for (int ks = 0; ks < TR::BQ / 16; ++ks)
                if (leader) umma_ts_f16(tmem_acc, tmem_a + bwd_pcol(ks, split_a(t)),
                            sdesc_join(b_lo_mn + ((split_b(t) * TR::Q_PANEL + ks * 2048) >> 4)), TR::IDESC_DKV,
                            (accumulate || (t | ks) != 0) ? 1u : 0u);
    }
}

// acc[D x 64 queries] = K^T dS^T with K MN-major (M = head dim) and dS^T MN-major (N = queries).
template <class TR>
__device__ __forceinline__ void bwd_issue_dq(uint32_t tmem_acc, uint32_t k_lo_mn, uint32_t ds_lo, bool leader) {
    if constexpr (!TR::SPLIT) {
#pragma unroll
        for (int ks = 0; ks < TR::BKV / 16; ++ks)
            if (leader) umma_ss_f16(tmem_acc, sdesc_join(k_lo_mn + ((ks * 2048) >> 4)), sdesc_join(ds_lo + ((ks * 2048) >> 4)), TR::IDESC_DQ, ks > 0);
    } else {
#pragma unroll
        for (int t = 0; t < 3; ++t)
#pragma unroll
            for (int ks = 0; ks < TR::BKV / 16; ++ks)
                if (leader) umma_ss_f16(tmem_acc, sdesc_join(k_lo_mn + ((split_a(t) * TR::KV_PANEL + ks * 2048) >> 4)),
                            sdesc_join(ds_lo + ((split_b(t) * TR::DS_PART + ks * 2048) >> 4)), TR::IDESC_DQ, (t | ks) != 0);
    }
}

template <bool V>
struct MaskedTag { static constexpr bool value = V; };

template <class TR>
__global__ void __launch_bounds__(TR::THREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_q_lo,
                const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_k_lo,
                const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_v_lo,
                const __grid_constant__ CUtensorMap tm_do, const __grid_constant__ CUtensorMap tm_do_lo,
                const __grid_constant__ CUtensorMap tm_dk, const __grid_constant__ CUtensorMap tm_dv,
                const __grid_constant__ CUtensorMap tm_dq, BwdParams prm) {
    constexpr int D = TR::D, BKV = TR::BKV, BQ = TR::BQ, NS = TR::NS;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint8_t* sK = smem + TR::OFF_K;
    uint8_t* sV = smem + TR::OFF_V;
    uint8_t* sQ = smem + TR::OFF_Q;
    uint8_t* sDO = smem + TR::OFF_DO;
    uint8_t* sDS = smem + TR::OFF_DS;
    float* sVec = reinterpret_cast<float*>(smem + TR::OFF_VEC);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + TR::OFF_BAR);
    uint64_t* kv_full = bars;               // [1]
    uint64_t* qdo_full = bars + 1;          // [NS]  TMA: Q, dO tiles + staged lse/delta
    uint64_t* qdo_empty = qdo_full + NS;    // [NS]  MMA commit: block consumed
    uint64_t* sdp_full = qdo_empty + NS;    // [2]   MMA commit: S^T and dP^T of a block are in TMEM
    uint64_t* pds_full = sdp_full + 2;      // [2]   compute warps: P^T, dS^T written (TMEM + smem)
    uint64_t* dq_full = pds_full + 2;       // [2]   MMA commit: dQ^T in TMEM (and the dS^T smem tile is free)
    uint64_t* dq_empty = dq_full + 2;       // [2]   drain warps: dQ^T copied to registers
    uint64_t* dkv_full = dq_empty + 2;      // [1]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(dkv_full + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int T = prm.T;
    const int bh = blockIdx.y;
    const int hd = bh % prm.H, bt = bh / prm.H;                 // head and batch coordinates
    const int n = blockIdx.x;                                   // key tile; tile 0 walks the most query blocks and starts first
    const int nqb = (T + BQ - 1) / BQ;
    const int m0 = prm.causal ? (n * BKV) / BQ : 0;             // first query block at or below the diagonal
    const int nblk = nqb - m0;
    AbortCtx ab{abort_flag, prm.status};

    if (tid == 0) {
        *abort_flag = 0;
        mbar_init(kv_full, 1);
        for (int s = 0; s < NS; ++s) { mbar_init(&qdo_full[s], 1); mbar_init(&qdo_empty[s], 1); }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&sdp_full[b], 1); mbar_init(&pds_full[b], 8);
            mbar_init(&dq_full[b], 1); mbar_init(&dq_empty[b], 4);
        }
        mbar_init(dkv_full, 1);
        fence_mbar_init();
    }
    if (warp == 13) { tmem_alloc(tmem_slot, TR::TM_COLS); tmem_relinquish(); }
    if (warp == 12 && lane == 0) {
        tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_k); tma_prefetch_desc(&tm_v); tma_prefetch_desc(&tm_do);
        tma_prefetch_desc(&tm_dk); tma_prefetch_desc(&tm_dv); tma_prefetch_desc(&tm_dq);
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
            mbar_arrive_expect_tx(kv_full, 2 * TR::KV_TILE);
            for (int p = 0; p < TR::NP; ++p) {
                const bool lo = TR::SPLIT && p;
                tma_load_4d(sK + p * TR::KV_PANEL, lo ? &tm_k_lo : &tm_k, kv_full, TR::SPLIT ? 0 : p * 64, n * BKV, hd, bt);
                tma_load_4d(sV + p * TR::KV_PANEL, lo ? &tm_v_lo : &tm_v, kv_full, TR::SPLIT ? 0 : p * 64, n * BKV, hd, bt);
            }
        }
        if (lane == 0) {
            for (int it = 0; it < nblk; ++it) {
                const int s = it % NS;
                const int m = m0 + it;
                mbar_wait(&qdo_empty[s], ((it / NS) & 1) ^ 1, ab, 10);
                mbar_arrive_expect_tx(&qdo_full[s], 2 * TR::Q_TILE + 2 * BQ * 4);
                for (int p = 0; p < TR::NP; ++p) {
                    const bool lo = TR::SPLIT && p;
                    tma_load_4d(sQ + s * TR::Q_TILE + p * TR::Q_PANEL, lo ? &tm_q_lo : &tm_q, &qdo_full[s], TR::SPLIT ? 0 : p * 64, m * BQ, hd, bt);
                    tma_load_4d(sDO + s * TR::Q_TILE + p * TR::Q_PANEL, lo ? &tm_do_lo : &tm_do, &qdo_full[s], TR::SPLIT ? 0 : p * 64, m * BQ, hd, bt);
                }
                // the block's 64 values of -lse*log2e and of -delta (padded rows, so always aligned and in range)
                const size_t voff = static_cast<size_t>(bh) * prm.T_pad + static_cast<size_t>(m) * BQ;
                bulk_load_1d(sVec + s * 2 * BQ, prm.nlse2 + voff, BQ * 4, &qdo_full[s]);
                bulk_load_1d(sVec + s * 2 * BQ + BQ, prm.ndelta + voff, BQ * 4, &qdo_full[s]);
            }
        }
    } else if (warp == 13) {
        // ------------------------------ MMA issuer ------------------------------
        // The whole warp walks the loop converged; only the MMA and commit instructions are predicated on one elected lane
        // (a converged warp issues an MMA every ~39 cycles and commits for free; a lone lane in a divergent branch pays
        // ~44 per MMA and ~44 more per commit).
        {
            const bool leader = elect_one_lane();
            // descriptor low words: K-major views (lbo unused = 16) and MN-major views (lbo = panel stride)
            const uint32_t lK = sdesc_lo(smem_u32(sK), 16), lV = sdesc_lo(smem_u32(sV), 16);
            const uint32_t lK_mn = sdesc_lo(smem_u32(sK), TR::KV_PANEL), lDS = sdesc_lo(smem_u32(sDS), 16);
            const uint32_t lQ0 = sdesc_lo(smem_u32(sQ), 16), lDO0 = sdesc_lo(smem_u32(sDO), 16);
            constexpr uint32_t kStage = TR::Q_TILE >> 4;                               // ring stage stride in descriptor units
            constexpr uint32_t kToMN = ((TR::Q_PANEL >> 4) << 16) - (1u << 16);        // K-major view -> MN-major view of a Q/dO stage
            mbar_wait(kv_full, 0, ab, 20);
            // S^T(blk) and dP^T(blk) into buffer blk & 1; the dP^T buffer must have been drained of dQ^T(blk - 2)
            auto issue_front = [&](int blk) {
                const int b = blk & 1, s = blk % NS;
                mbar_wait(&qdo_full[s], (blk / NS) & 1, ab, 21);
                tc_fence_after_sync();
                bwd_issue_kmajor<TR>(tmem + TR::TM_ST + b * 64, lK, lQ0 + s * kStage, leader);
                if (blk >= 2) { mbar_wait(&dq_empty[b], ((blk - 2) >> 1) & 1, ab, 24); tc_fence_after_sync(); }
                bwd_issue_kmajor<TR>(tmem + TR::TM_DP + b * 64, lV, lDO0 + s * kStage, leader);
                if (leader) umma_commit(&sdp_full[b]);
            };
            issue_front(0);
            if (nblk > 1) issue_front(1);
            for (int it = 0; it < nblk; ++it) {
                const int b = it & 1, s = it % NS;
                const uint32_t lQ_mn = lQ0 + s * kStage + kToMN, lDO_mn = lDO0 + s * kStage + kToMN;
                const uint32_t t_st = tmem + TR::TM_ST + b * 64, t_dp = tmem + TR::TM_DP + b * 64;
                mbar_wait(&pds_full[b], (it >> 1) & 1, ab, 22);
                tc_fence_after_sync();
                if constexpr (!TR::SPLIT) {
                    bwd_issue_dq<TR>(t_dp, lK_mn, lDS, leader);                            // dQ^T(it) over the consumed dP^T buffer
                    if (leader) umma_commit(&dq_full[b]);
                    bwd_issue_acc<TR>(tmem + TR::TM_DK, t_st, 1, lQ_mn, it > 0, leader);   // dK += dS^T Q
                    bwd_issue_acc<TR>(tmem + TR::TM_DV, t_st, 0, lDO_mn, it > 0, leader);  // dV += P^T dO
                } else {
                    bwd_issue_acc<TR>(tmem + TR::TM_DV, t_st, 0, lDO_mn, it > 0, leader);
                    bwd_issue_acc<TR>(tmem + TR::TM_DK, t_dp, 0, lQ_mn, it > 0, leader);
                    bwd_issue_dq<TR>(t_dp, lK_mn, lDS, leader);
                    if (leader) umma_commit(&dq_full[b]);
                }
                if (leader) umma_commit(&qdo_empty[s]);
                if (it + 2 < nblk) issue_front(it + 2);
            }
            if (leader) umma_commit(dkv_full);
        }
    } else if (warp < 8) {
        // ------------------------------ compute: P^T and dS^T ------------------------------
        asm volatile("setmaxnreg.inc.sync.aligned.u32 160;");
        const int h = warp >> 2;                     // which 32 query columns
        const int wq = warp & 3;
        const int r = wq * 32 + lane;                // key row inside the tile
        const int kv_g = n * BKV + r;
        const bool row_dead = kv_g >= T;
        const bool tail_tile = (n + 1) * BKV > T;     // this key tile has rows past T
        const uint32_t lane_base = static_cast<uint32_t>(wq * 32) << 16;
        const float c = prm.scale_log2;

        for (int it = 0; it < nblk; ++it) {
            const int b = it & 1, s = it % NS, m = m0 + it;
            const float* v_lse = sVec + s * 2 * BQ + h * 32;
            const float* v_del = v_lse + BQ;
            const uint32_t t_st = tmem + TR::TM_ST + b * 64 + h * 32 + lane_base;
            const uint32_t t_dp = tmem + TR::TM_DP + b * 64 + h * 32 + lane_base;
            mbar_wait(&qdo_full[s], (it / NS) & 1, ab, 30);      // lse / delta visible
            mbar_wait(&sdp_full[b], (it >> 1) & 1, ab, 31);
            tc_fence_after_sync();
            uint32_t sr[32], dr[32];
            tmem_ld_x32(t_st, sr);
            tmem_ld_x32(t_dp, dr);
            tmem_wait_ld();
            const bool diag = prm.causal && (m * BQ < (n + 1) * BKV);
            const int q0 = m * BQ + h * 32;
            const bool masked = diag || tail_tile;             // uniform per block: most blocks take the unmasked path
            uint32_t pk[16], dk[16], pl[16], dl[16];
            const uint64_t c2 = pack_f32x2(c, c);
            const float4* v_lse4 = reinterpret_cast<const float4*>(v_lse);
            const float4* v_del4 = reinterpret_cast<const float4*>(v_del);
            // The masked and the unmasked block are two copies of the loop: a branch inside the loop body would cut it
            // into one basic block per element pair and expose the full FFMA -> MUFU -> convert latency 16 times.
            auto body = [&](auto masked_tag) {
                constexpr bool kMasked = decltype(masked_tag)::value;
#pragma unroll
                for (int e4 = 0; e4 < 8; ++e4) {
                    const float4 nl = v_lse4[e4], nd = v_del4[e4];   // broadcast 16-byte loads: 4 query columns each
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        const int e = e4 * 4 + half * 2;
                        const uint64_t nl2 = half ? pack_f32x2(nl.z, nl.w) : pack_f32x2(nl.x, nl.y);
                        const uint64_t nd2 = half ? pack_f32x2(nd.z, nd.w) : pack_f32x2(nd.x, nd.y);
                        float x0, x1;
                        unpack_f32x2(ffma2(pack_f32x2(__uint_as_float(sr[e]), __uint_as_float(sr[e + 1])), c2, nl2), x0, x1);
                        float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
                        if constexpr (kMasked) {
                            if (row_dead || (diag && kv_g > q0 + e)) p0 = 0.f;
                            if (row_dead || (diag && kv_g > q0 + e + 1)) p1 = 0.f;
                        }
                        const uint64_t p2 = pack_f32x2(p0, p1);
                        float d0, d1;
                        unpack_f32x2(fmul2(p2, fadd2(pack_f32x2(__uint_as_float(dr[e]), __uint_as_float(dr[e + 1])), nd2)), d0, d1);
                        pk[e >> 1] = pack_bf16x2(p0, p1);
                        dk[e >> 1] = pack_bf16x2(d0, d1);
                        if constexpr (TR::SPLIT) {
                            pl[e >> 1] = pack_bf16x2(p0 - __uint_as_float(pk[e >> 1] << 16), p1 - __uint_as_float(pk[e >> 1] & 0xffff0000u));
                            dl[e >> 1] = pack_bf16x2(d0 - __uint_as_float(dk[e >> 1] << 16), d1 - __uint_as_float(dk[e >> 1] & 0xffff0000u));
                        }
                    }
                }
            };
            if (masked) body(MaskedTag<true>{}); else body(MaskedTag<false>{});
            tmem_st_x16(t_st, pk);
            if constexpr (!TR::SPLIT) {
                tmem_st_x16(t_st + 16, dk);
            } else {
                tmem_st_x16(t_st + 16, pl);
                tmem_st_x16(t_dp, dk);
                tmem_st_x16(t_dp + 16, dl);
            }
            // the single dS^T smem tile is free once dQ^T of the previous block has completed
            if (it >= 1) mbar_wait(&dq_full[(it - 1) & 1], ((it - 1) >> 1) & 1, ab, 32);
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4) {
                st_shared_sw128(sDS, r, h * 4 + c4, make_uint4(dk[4 * c4], dk[4 * c4 + 1], dk[4 * c4 + 2], dk[4 * c4 + 3]));
                if constexpr (TR::SPLIT)
                    st_shared_sw128(sDS + TR::DS_PART, r, h * 4 + c4, make_uint4(dl[4 * c4], dl[4 * c4 + 1], dl[4 * c4 + 2], dl[4 * c4 + 3]));
            }
            tmem_wait_st();
            fence_proxy_async_smem();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&pds_full[b]);
        }

        // ---- epilogue: warps 0-3 write dV, warps 4-7 write dK (scaled) ----
        mbar_wait(dkv_full, 0, ab, 33);
        tc_fence_after_sync();
        {
            const uint32_t t_acc = tmem + (h ? TR::TM_DK : TR::TM_DV) + lane_base;
            const float mul = h ? prm.scale : 1.f;
            uint8_t* stage = sQ + h * TR::OUT_TILE;
#pragma unroll
            for (int cc = 0; cc < D; cc += 32) {
                uint32_t rr[32];
                tmem_ld_x32(t_acc + cc, rr);
                tmem_wait_ld();
                if constexpr (!TR::SPLIT) {
                    const int panel = cc / 64, chunk0 = (cc % 64) / 8;
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        uint4 v;
                        v.x = pack_bf16x2(__uint_as_float(rr[q4 * 8 + 0]) * mul, __uint_as_float(rr[q4 * 8 + 1]) * mul);
                        v.y = pack_bf16x2(__uint_as_float(rr[q4 * 8 + 2]) * mul, __uint_as_float(rr[q4 * 8 + 3]) * mul);
                        v.z = pack_bf16x2(__uint_as_float(rr[q4 * 8 + 4]) * mul, __uint_as_float(rr[q4 * 8 + 5]) * mul);
                        v.w = pack_bf16x2(__uint_as_float(rr[q4 * 8 + 6]) * mul, __uint_as_float(rr[q4 * 8 + 7]) * mul);
                        st_shared_sw128(stage + panel * TR::KV_PANEL, r, chunk0 + q4, v);
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
                        st_shared_sw128(stage + panel * TR::KV_PANEL, r, q4, v);
                    }
                }
            }
            fence_proxy_async_smem();
            asm volatile("bar.sync %0, 128;" ::"r"(1 + h) : "memory");
            if ((tid & 127) == 0) {
                for (int p = 0; p < TR::OUT_PANELS; ++p)
                    tma_store_4d(h ? &tm_dk : &tm_dv, stage + p * TR::KV_PANEL, p * TR::OUT_PANEL_ELEMS, n * BKV, hd, bt);
                tma_store_commit();
                tma_store_wait_read_all();     // the CTA may leave once its shared memory has been read; the writes complete on their own
            }
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
        for (int it = 0; it < nblk; ++it) {
            const int b = it & 1, m = m0 + it;
            mbar_wait(&dq_full[b], (it >> 1) & 1, ab, 40);
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
                for (int e = 0; e < 32; ++e) stage[e * D + d] = __uint_as_float(r0[e]);
#pragma unroll
                for (int e = 0; e < 32; ++e) stage[(32 + e) * D + d] = __uint_as_float(r1[e]);
            }
            fence_proxy_async_smem();
            asm volatile("bar.sync 3, 128;" ::: "memory");
            if (issuer) {
                tma_reduce_add_3d(&tm_dq, stage, 0, m * BQ, bh);    // rows past T are clipped
                tma_store_commit();
            }
        }
        if (issuer) tma_store_wait_read_all();     // the CTA may leave once its shared memory has been read; the writes complete on their own
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
