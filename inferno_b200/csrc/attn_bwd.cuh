// Causal flash-attention backward for sm_100a: block algorithm, traits and MMA issue helpers.  The kernel itself
// (persistent CTAs walking a work-item list) is attn_bwd_persist_kernel in attn_bwd_persist.cuh.
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
// A work item is one 128-row key/value tile of one (batch, head); the CTA walks the
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
// Software pipeline of the MMA issuer inside an item (block = one 64-row query block, b = block % NB; NB = 2 below):
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
    // S^T / dP^T buffers in TMEM = query blocks in flight.  Head dim 128 fills the 512 columns with two; bf16 head dim 64
    // leaves 128 columns over, which buy a third (the compute warps, not the tensor pipe, pace a block there, and with
    // three blocks in flight their chain front -> P^T / dS^T -> back overlaps itself).  The split mode has the columns
    // but not the shared memory for the fourth ring stage a third buffer needs.
    static constexpr int NB = (D == 64 && !SPLIT) ? 3 : 2;
    static constexpr int NS = NB + 1;                        // Q/dO ring depth: the blocks in flight plus the one being loaded
    static constexpr int NTERMS = SPLIT ? 3 : 1;
    static constexpr int OUT_TILE = SPLIT ? BKV * D * 4 : KV_TILE;   // dK / dV staging bytes
    static constexpr int OUT_PANELS = SPLIT ? 2 : D / 64;
    static constexpr int OUT_PANEL_ELEMS = SPLIT ? 32 : 64;
    static constexpr uint32_t IDESC_ST = make_idesc(kFmtBF16, BKV, BQ, kMajorK, kMajorK);
    static constexpr uint32_t IDESC_DKV = make_idesc(kFmtBF16, BKV, D, kMajorK, kMajorMN);
    static constexpr uint32_t IDESC_DQ = make_idesc(kFmtBF16, D, BQ, kMajorMN, kMajorMN);
    static constexpr uint32_t TM_ST = 0, TM_DP = NB * 64, TM_DV = 2 * NB * 64, TM_DK = TM_DV + D, TM_COLS = 512;
    static_assert(TM_DK + D <= TM_COLS, "TMEM budget");
    static constexpr int OFF_K = 0;
    static constexpr int OFF_V = OFF_K + KV_TILE;
    static constexpr int OFF_Q = OFF_V + KV_TILE;            // NS tiles
    static constexpr int OFF_DO = OFF_Q + NS * Q_TILE;       // NS tiles
    static constexpr int OFF_DS = OFF_DO + NS * Q_TILE;      // one dS^T tile (hi + lo in split mode)
    static constexpr int OFF_DQ = OFF_DS + DS_TILE;          // dQ staging [64 queries x D] fp32, row-major, for the TMA reduction
    static constexpr int DQ_STAGE = BQ * D * 4;
    // the persistent kernel's drain warps also stage the dK / dV tile here: the region holds whichever is larger
    static constexpr int DQ_REGION = DQ_STAGE > OUT_TILE ? DQ_STAGE : OUT_TILE;
    static constexpr int OFF_VEC = OFF_DQ + DQ_REGION;    // NS x (lse[64], delta[64]) floats
    static constexpr int OFF_BAR = OFF_VEC + NS * 2 * BQ * 4;
    static constexpr int SMEM_BYTES = OFF_BAR + 512 + 1024;
    static constexpr int THREADS = 512;
    static_assert(SMEM_BYTES <= 232448, "shared memory budget");
};

struct BwdParams {
    const float* nlse2;    // [BH, T_pad]  -lse * log2(e), 0 in the padding
    const float* ndelta;   // [BH, T_pad]  -rowsum(dO * O), 0 in the padding
    int T_pad;             // T rounded up to a multiple of 64
    int* status;
    int T, BH, H, causal;  // H: heads per batch entry (operand tensor maps are 4-D: column, token, head, batch)
    float scale, scale_log2;
    float dq_scale;        // factor applied to every dQ^T partial before it is added: 1 when an fp32 accumulator is finished by
                           // dq_finish_kernel, `scale` when the partials go straight into a dense fp32 dQ (fp32 I/O)
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

}  // namespace ib200
