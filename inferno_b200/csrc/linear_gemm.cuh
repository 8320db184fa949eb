// bf16 GEMM with fp32 accumulation and an optional bias epilogue for sm_100a: the projections either side of
// attention (qkv = x Wqkv + b before it, y W_out + b after it).
//
// Replaces, for those two layers, the reference's Linear::forward = matmul(x, W) + b
// (src/inferno/modules/linear.cpp:99-106 -> cublas_mm_row_major, src/inferno/cuda/cudamatmul.cu:1058-1112, plus the
// broadcast add kernel, src/inferno/cuda/cudaadd.cu:20-142) and, through the operand-major flags, the two GEMMs of its
// backward, MMBackward (src/inferno/gradfn/mmbackward.cpp:36-98): dX = dY W^T and dW = X^T dY.  The reference
// materialises every transpose with a copy kernel; here a transposed operand is only a different shared-memory
// descriptor (MN-major instead of K-major).
//
//   C[M, N] = A[M, K] * B[K, N] (+ bias[N])
//   A_MN = false: A stored [M rows, K contiguous]        A_MN = true: A stored [K rows, M contiguous]  (A = X^T)
//   B_MN = true : B stored [K rows, N contiguous]        B_MN = false: B stored [N rows, K contiguous] (B = W^T)
//
// Persistent CTAs (one per SM) walk 128 x 256 output tiles.  Warp 4 streams A / B k-slices of 64 through a 4-stage TMA
// ring, one lane of warp 5 issues 128x256x16 tcgen05 MMAs into one of two 256-column TMEM accumulators, and warps 0-3
// drain the other accumulator (TMEM -> registers -> +bias -> bf16 -> swizzled smem -> TMA store), so the epilogue of a
// tile overlaps the main loop of the next.
//
// Split-K (GemmParams::splits > 1) is for outputs with fewer tiles than SMs and a long K, the weight gradient
// dW = X^T dY of a projection: the work unit becomes (tile, K slab), every unit adds its partial tile, rounded to bf16,
// into the zeroed output with a TMA reduction.  The output then carries one bf16 rounding per slab instead of one in
// all (relative error about 2^-9 * sqrt(slabs + 1)), which is the price of needing no fp32 workspace.
#pragma once

#include "sm100_ptx.cuh"

namespace ib200 {

struct GemmTraits {
    static constexpr int BM = 128, BN = 256, BK = 64;
    static constexpr int STAGES = 4;
    static constexpr int A_BYTES = BM * BK * 2;                  // 16 KB
    static constexpr int B_BYTES = BN * BK * 2;                  // 32 KB
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int OUT_CHUNK_COLS = 64;                    // epilogue staging: [128 rows x 64 cols] bf16 = one 128B-swizzled panel
    static constexpr int OUT_CHUNK_BYTES = BM * 128;
    static constexpr int OFF_OUT = STAGES * STAGE_BYTES;         // one staging panel
    static constexpr int OFF_BIAS = OFF_OUT + OUT_CHUNK_BYTES;   // 2 x 256 floats (per accumulator buffer)
    static constexpr int OFF_BAR = OFF_BIAS + 2 * BN * 4;
    static constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;
    static constexpr int THREADS = 192;                          // 4 epilogue warps + TMA warp + MMA warp
    static constexpr uint32_t TM_COLS = 512;
    static_assert(SMEM_BYTES <= 232448, "shared memory budget");
};

struct GemmParams {
    const float* bias;     // [N] fp32 or null
    int M, N, K;
    int splits;            // >1: the K range is cut into this many slabs; each (tile, slab) unit adds its bf16 partial tile into a zeroed C
    int* status;
};

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(GemmTraits::THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                 const __grid_constant__ CUtensorMap tm_c, GemmParams prm) {
    using TR = GemmTraits;
    constexpr int BM = TR::BM, BN = TR::BN, BK = TR::BK, NS = TR::STAGES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint8_t* sOut = smem + TR::OFF_OUT;
    float* sBias = reinterpret_cast<float*>(smem + TR::OFF_BIAS);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + TR::OFF_BAR);
    uint64_t* full = bars;                  // [NS]  TMA -> MMA
    uint64_t* empty = full + NS;            // [NS]  MMA -> TMA
    uint64_t* acc_full = empty + NS;        // [2]   MMA -> epilogue
    uint64_t* acc_empty = acc_full + 2;     // [2]   epilogue -> MMA
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tiles_m = (prm.M + BM - 1) / BM, tiles_n = (prm.N + BN - 1) / BN;
    const int n_tiles = tiles_m * tiles_n;
    const int k_slices = (prm.K + BK - 1) / BK;
    const int splits = prm.splits > 1 ? prm.splits : 1;
    const int n_units = n_tiles * splits;                       // unit u: tile u % n_tiles, K slab u / n_tiles
    const int k_per = (k_slices + splits - 1) / splits;
    AbortCtx ab{abort_flag, prm.status};

    if (tid == 0) {
        *abort_flag = 0;
        for (int s = 0; s < NS; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4); }
        fence_mbar_init();
    }
    if (warp == 5) { tmem_alloc(tmem_slot, TR::TM_COLS); tmem_relinquish(); }
    if (warp == 4 && lane == 0) { tma_prefetch_desc(&tm_a); tma_prefetch_desc(&tm_b); tma_prefetch_desc(&tm_c); }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    if (warp == 4) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            int it = 0;     // running k-slice count across tiles: ring position
            for (int unit = blockIdx.x; unit < n_units; unit += gridDim.x) {
                const int tile = unit % n_tiles, ks0 = (unit / n_tiles) * k_per, ks1 = min(k_slices, ks0 + k_per);
                const int m0 = (tile % tiles_m) * BM, n0 = (tile / tiles_m) * BN;
                for (int ks = ks0; ks < ks1; ++ks, ++it) {
                    const int s = it % NS;
                    mbar_wait(&empty[s], ((it / NS) & 1) ^ 1, ab, 10);
                    mbar_arrive_expect_tx(&full[s], TR::STAGE_BYTES);
                    uint8_t* sa = smem + s * TR::STAGE_BYTES;
                    uint8_t* sb = sa + TR::A_BYTES;
                    const int k0 = ks * BK;
                    if constexpr (!A_MN) {
                        tma_load_3d(sa, &tm_a, &full[s], k0, m0, 0);                       // [128 m-rows x 64 k]
                    } else {
                        tma_load_3d(sa, &tm_a, &full[s], m0, k0, 0);                       // two panels [64 k-rows x 64 m]
                        tma_load_3d(sa + BK * 128, &tm_a, &full[s], m0 + 64, k0, 0);
                    }
                    if constexpr (!B_MN) {
                        tma_load_3d(sb, &tm_b, &full[s], k0, n0, 0);                       // [256 n-rows x 64 k]
                    } else {
                        for (int p = 0; p < BN / 64; ++p)                                  // four panels [64 k-rows x 64 n]
                            tma_load_3d(sb + p * BK * 128, &tm_b, &full[s], n0 + p * 64, k0, 0);
                    }
                }
            }
        }
    } else if (warp == 5) {
        // ------------------------------ MMA issuer ------------------------------
        // The warp stays converged; only the MMA / commit instructions are predicated on one elected lane (commits are
        // then free, where a lone lane in a divergent branch pays ~44 cycles of tensor-pipe time for each).
        {
            const bool leader = elect_one_lane();
            constexpr uint32_t idesc = make_idesc(kFmtBF16, BM, BN, A_MN ? kMajorMN : kMajorK, B_MN ? kMajorMN : kMajorK);
            int it = 0, tcount = 0;
            for (int unit = blockIdx.x; unit < n_units; unit += gridDim.x, ++tcount) {
                const int ks0 = (unit / n_tiles) * k_per, ks1 = min(k_slices, ks0 + k_per);
                const int buf = tcount & 1;
                mbar_wait(&acc_empty[buf], (((tcount >> 1) & 1) ^ 1), ab, 20);             // epilogue has drained this accumulator
                tc_fence_after_sync();
                for (int ks = ks0; ks < ks1; ++ks, ++it) {
                    const int s = it % NS;
                    mbar_wait(&full[s], (it / NS) & 1, ab, 21);
                    tc_fence_after_sync();
                    const uint32_t sa = smem_u32(smem + s * TR::STAGE_BYTES), sb = sa + TR::A_BYTES;
                    const uint32_t a_lo = sdesc_lo(sa, A_MN ? BK * 128 : 16), b_lo = sdesc_lo(sb, B_MN ? BK * 128 : 16);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {
                        const uint32_t ao = A_MN ? (k * 2048) >> 4 : (k * 32) >> 4;
                        const uint32_t bo = B_MN ? (k * 2048) >> 4 : (k * 32) >> 4;
                        if (leader) umma_ss_f16(tmem + buf * BN, sdesc_join(a_lo + ao), sdesc_join(b_lo + bo), idesc, ((ks - ks0) | k) != 0);
                    }
                    if (leader) umma_commit(&empty[s]);
                }
                if (leader) umma_commit(&acc_full[buf]);
            }
        }
    } else {
        // ------------------------------ epilogue (warps 0-3: one thread per output row) ------------------------------
        const int r = tid;                                           // row inside the tile == TMEM lane
        const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
        int tcount = 0;
        for (int unit = blockIdx.x; unit < n_units; unit += gridDim.x, ++tcount) {
            const int tile = unit % n_tiles;
            const bool first_slab = unit < n_tiles;                   // the bias goes in once
            const int buf = tcount & 1;
            const int m0 = (tile % tiles_m) * BM, n0 = (tile / tiles_m) * BN;
            // stage this tile's bias slice (zeros where there is no bias or past N)
            float* bias_s = sBias + buf * BN;
            for (int c = tid; c < BN; c += 128) bias_s[c] = (prm.bias && first_slab && n0 + c < prm.N) ? prm.bias[n0 + c] : 0.f;
            asm volatile("bar.sync 1, 128;" ::: "memory");
            mbar_wait(&acc_full[buf], (tcount >> 1) & 1, ab, 30);
            tc_fence_after_sync();
#pragma unroll 1
            for (int ch = 0; ch < BN / TR::OUT_CHUNK_COLS; ++ch) {
                uint8_t* stage = sOut;
                // the TMA store of the previous chunk must have finished reading the staging panel
                if (tid == 0) tma_store_wait_read_all();
                asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    uint32_t v[32];
                    tmem_ld_x32(tmem + buf * BN + ch * 64 + half * 32 + lane_base, v);
                    tmem_wait_ld();
                    const float* bs = bias_s + ch * 64 + half * 32;
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        uint4 o;
                        o.x = pack_bf16x2(__uint_as_float(v[q4 * 8 + 0]) + bs[q4 * 8 + 0], __uint_as_float(v[q4 * 8 + 1]) + bs[q4 * 8 + 1]);
                        o.y = pack_bf16x2(__uint_as_float(v[q4 * 8 + 2]) + bs[q4 * 8 + 2], __uint_as_float(v[q4 * 8 + 3]) + bs[q4 * 8 + 3]);
                        o.z = pack_bf16x2(__uint_as_float(v[q4 * 8 + 4]) + bs[q4 * 8 + 4], __uint_as_float(v[q4 * 8 + 5]) + bs[q4 * 8 + 5]);
                        o.w = pack_bf16x2(__uint_as_float(v[q4 * 8 + 6]) + bs[q4 * 8 + 6], __uint_as_float(v[q4 * 8 + 7]) + bs[q4 * 8 + 7]);
                        st_shared_sw128(stage, r, half * 4 + q4, o);
                    }
                }
                if (ch == BN / TR::OUT_CHUNK_COLS - 1) {
                    // every column of the accumulator has been read: hand it back to the MMA warp
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&acc_empty[buf]);
                }
                fence_proxy_async_smem();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (tid == 0) {
                    if (splits > 1) tma_reduce_add_3d(&tm_c, stage, n0 + ch * 64, m0, 0);   // bf16 add into the zeroed output
                    else tma_store_3d(&tm_c, stage, n0 + ch * 64, m0, 0);                   // rows / columns past M / N are clipped
                    tma_store_commit();
                }
            }
        }
        if (tid == 0) tma_store_wait_read_all();     // the CTA may leave once its shared memory has been read; the writes complete on their own
    }

    tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag != 0) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    if (warp == 5) tmem_dealloc(tmem, TR::TM_COLS);
}

// Column sums of a [M, N] bf16 matrix into fp32 (bias gradient: the reference's sum_to_shape after the broadcast add,
// src/inferno/core/broadcastops.cpp).  Block (x, y): 64 columns, rows y * rows_per_block ...; 256 threads = 8 row-groups
// x 32 column-pairs; the row slabs are combined with fp32 atomics into `out`, which the host zeroes first.
__global__ void __launch_bounds__(256) colsum_bf16_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ out, int M, int N,
                                                          int rows_per_block) {
    __shared__ float2 part[8][32];
    const int cp = threadIdx.x & 31, rg = threadIdx.x >> 5;
    const int col = blockIdx.x * 64 + cp * 2;
    const int row0 = blockIdx.y * rows_per_block, row1 = min(M, row0 + rows_per_block);
    float2 acc = make_float2(0.f, 0.f);
    if (col < N) {
        for (int row = row0 + rg; row < row1; row += 8) {
            const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(x + static_cast<size_t>(row) * N + col);
            const float2 f = __bfloat1622float2(v);
            acc.x += f.x;
            acc.y += f.y;
        }
    }
    part[rg][cp] = acc;
    __syncthreads();
    if (rg == 0 && col < N) {
        float2 s = part[0][cp];
#pragma unroll
        for (int i = 1; i < 8; ++i) { s.x += part[i][cp].x; s.y += part[i][cp].y; }
        atomicAdd(out + col, s.x);
        if (col + 1 < N) atomicAdd(out + col + 1, s.y);
    }
}

}  // namespace ib200
