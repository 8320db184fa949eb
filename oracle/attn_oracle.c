/* TEST INFRASTRUCTURE ONLY -- a CPU restatement of the reference's causal
 * attention path, used as the checker in tests/, in the smoke test and as the
 * "port" CPU baseline.  The shipped library never links or calls this file.
 *
 * Parity pin: the reference has no live tests and no golden vectors for this
 * path, so this restatement is pinned against the reference's OWN code compiled
 * from its sources (oracle/_ref/ref_attention) -- bit-exact on the committed
 * fixtures under tests/golden/ -- and against an independent fp64 evaluation.
 *
 * Each step keeps the reference's arithmetic: fp32 everywhere, sequential
 * accumulation in the same loop order, scale applied as a separate fp32
 * multiply before masking, mask value -1e9, exp evaluated in double.
 * Citations are paths inside the reference project.
 */
#include <math.h>
#include <stddef.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* C[M,N] = A[M,K] * B[K,N], fp32 sequential sum over k.
 * src/inferno/core/cpuops.h:336-434 (cpu_matmul: m, n, k loops, RT sum). */
static void mm(const float* a, const float* b, float* c, size_t M, size_t K, size_t N) {
    for (size_t m = 0; m < M; ++m)
        for (size_t n = 0; n < N; ++n) {
            float sum = 0.0f;
            for (size_t k = 0; k < K; ++k) sum += a[m * K + k] * b[k * N + n];
            c[m * N + n] = sum;
        }
}

/* dst[C,R] = src[R,C]^T  -- transpose(-1,-2).contiguous()
 * (src/inferno/core/ops.cpp:750-785 view + :1302-1342 dense copy). */
static void transpose(const float* src, float* dst, size_t R, size_t C) {
    for (size_t r = 0; r < R; ++r)
        for (size_t c = 0; c < C; ++c) dst[c * R + r] = src[r * C + c];
}

/* One (batch, head) slice, forward.  p_out (T*T) and s1_out (T*T) are kept for
 * the backward.  InfernoApp/main.cpp:737-754. */
static void head_forward(const float* q, const float* k, const float* v, float* o,
                         float* p, float* kt, size_t T, size_t D, float scale) {
    transpose(k, kt, T, D);                 /* main.cpp:737 */
    mm(q, kt, p, T, D, T);                  /* main.cpp:740, scores = q @ kt */
    for (size_t i = 0; i < T * T; ++i)      /* main.cpp:743-744 -> cpuops.h:165-226 (cpu_multiply) */
        p[i] = p[i] * scale;
    for (size_t i = 0; i < T; ++i)          /* triu(ones,1): cpuops.h:617-656; masked_fill: cpuops.h:659-705 */
        for (size_t j = i + 1; j < T; ++j) p[i * T + j] = -1e9f;
    for (size_t i = 0; i < T; ++i) {        /* src/inferno/functional/softmax_kernels.h:40-104 */
        float* row = p + i * T;
        float mx = -3.402823466e+38f;       /* numeric_limits<float>::lowest() */
        for (size_t j = 0; j < T; ++j) if (row[j] > mx) mx = row[j];
        float sum = 0.0f;
        for (size_t j = 0; j < T; ++j) {
            float e = (float)exp((double)(row[j] - mx));
            row[j] = e;
            sum += e;
        }
        for (size_t j = 0; j < T; ++j) row[j] /= sum;
    }
    mm(p, v, o, T, T, D);                   /* main.cpp:754, y = attn @ v */
}

/* One (batch, head) slice, backward, given P from the forward.
 * Node order: MMBackward(attn,v) -> SoftmaxBackward -> MultiplyBackward(scale)
 * -> MMBackward(q,kt) -> ContiguousBackward/TransposeBackward. */
static void head_backward(const float* q, const float* k, const float* v, const float* dO,
                          const float* p, const float* kt, float* dq, float* dk, float* dv,
                          float* dp, float* tmpTT, float* tmpTD, size_t T, size_t D, float scale) {
    /* src/inferno/gradfn/mmbackward.cpp:76-80: dA = G @ B^T ; dB = A^T @ G */
    transpose(v, tmpTD, T, D);              /* v^T : [D,T] */
    mm(dO, tmpTD, dp, T, D, T);             /* dP = dO @ V^T */
    transpose(p, tmpTT, T, T);              /* P^T */
    mm(tmpTT, dO, dv, T, T, D);             /* dV = P^T @ dO */
    /* src/inferno/gradfn/softmaxbackward.h:64-131: dot = sum(g*y); dx = y*(g-dot) */
    for (size_t i = 0; i < T; ++i) {
        float dot = 0.0f;
        for (size_t j = 0; j < T; ++j) dot += dp[i * T + j] * p[i * T + j];
        for (size_t j = 0; j < T; ++j) {
            float y = p[i * T + j], g = dp[i * T + j];
            dp[i * T + j] = y * (g - dot);
        }
    }
    /* The masked_fill output is the stage boundary (no backward node exists in
     * the reference, ops.cpp:1235-1289); dS is exactly 0 where masked since P=0.
     * src/inferno/gradfn/multiplybackward.cpp:34-57: g * scale. */
    for (size_t i = 0; i < T * T; ++i) dp[i] = dp[i] * scale;
    /* MMBackward(q, kt): dQ = dS @ kt^T = dS @ K ; d(kt) = Q^T @ dS, then the
     * transpose backward maps d(kt)[D,T] to dK[T,D]. */
    transpose(kt, tmpTD, D, T);             /* kt^T = K as a dense copy */
    mm(dp, tmpTD, dq, T, T, D);
    transpose(q, tmpTD, T, D);              /* Q^T : [D,T] */
    float* dkt = tmpTT;                     /* reuse: needs D*T <= T*T or separate buffer */
    mm(tmpTD, dp, dkt, D, T, T);
    transpose(dkt, dk, D, T);
}

/* Dense row-major [B,H,T,D] fp32 in and out.  want_bwd=0 skips gradients.
 * Heads are independent; with OpenMP they run on `threads` host threads
 * (0 = all).  Returns 0, or -1 if scratch allocation failed. */
int attn_oracle_f32(const float* q, const float* k, const float* v, const float* dO,
                    float* o, float* dq, float* dk, float* dv,
                    long B, long H, long T, long D, float scale, int want_bwd, int threads) {
    const long BH = B * H;
    int failed = 0;
#ifdef _OPENMP
    if (threads > 0) omp_set_num_threads(threads);
#endif
#pragma omp parallel for schedule(dynamic, 1)
    for (long bh = 0; bh < BH; ++bh) {
        const size_t TT = (size_t)T * (size_t)(T > D ? T : D), TD = (size_t)T * D;
        float* p = (float*)malloc(sizeof(float) * TT);
        float* kt = (float*)malloc(sizeof(float) * TD);
        float* dp = want_bwd ? (float*)malloc(sizeof(float) * TT) : NULL;
        float* tTT = want_bwd ? (float*)malloc(sizeof(float) * TT) : NULL;
        float* tTD = want_bwd ? (float*)malloc(sizeof(float) * TD) : NULL;
        if (!p || !kt || (want_bwd && (!dp || !tTT || !tTD))) {
            failed = 1;
        } else {
            const size_t off = (size_t)bh * TD;
            head_forward(q + off, k + off, v + off, o + off, p, kt, (size_t)T, (size_t)D, scale);
            if (want_bwd)
                head_backward(q + off, k + off, v + off, dO + off, p, kt, dq + off, dk + off, dv + off,
                              dp, tTT, tTD, (size_t)T, (size_t)D, scale);
        }
        free(p); free(kt); free(dp); free(tTT); free(tTD);
    }
    return failed ? -1 : 0;
}

int attn_oracle_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
