// Causal flash-attention forward for sm_100a: tile algorithm, traits and MMA issue helpers.  The kernel itself
// (persistent CTAs walking a work-item list) is attn_fwd_persist_kernel in attn_fwd_persist.cuh.
//
// Replaces the reference's composed forward
//   matmul(q,kt) -> * scale -> triu/masked_fill(-1e9) -> Softmax -> matmul(attn,v)
// (InfernoApp/main.cpp:737-754; ops in src/inferno/core/ops.cpp:437-735, 204-270,
// 1235-1289, 1355-1398; src/inferno/functional/softmax.cpp:22-79) with one kernel
// that never materialises the [T,T] score matrix and saves the per-row
// log-sum-exp for the backward pass.
//
// A work item is two adjacent 128-row query tiles of one (batch, head); the CTA walks the
// key/value tiles up to the diagonal:
//   warps 10-11 idle (they only donate registers)
//   warp 9      TMA producer: the Q tiles and K_0 once per item, then one load group {K_{j+1}, V_j}
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

}  // namespace ib200
