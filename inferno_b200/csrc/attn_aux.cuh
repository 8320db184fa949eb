// Bandwidth-bound helper kernels around the attention main kernels:
//   * split_bf16   fp32 x -> (hi, lo) bf16 pair with hi = bf16(x), lo = bf16(x - hi); the
//                  fp32-I/O kernels multiply such pairs in three bf16 MMAs
//   * bwd_prepass  one launch ahead of the backward main kernel: -delta[row] = -sum_d O[row,d] * dO[row,d] (and
//                  -lse*log2e beside it), the zeroing of the dQ accumulator, the workspace header and (fp32 I/O) the
//                  operand splits; delta is the reference's
//                  dot = sum_j dP_ij P_ij (src/inferno/gradfn/softmaxbackward.h:101-109)
//                  rewritten so that it needs no [T,T] matrix
//   * dq_finish    dQ = scale * accumulator, cast to the output type; the scale is
//                  the reference's MultiplyBackward (src/inferno/gradfn/multiplybackward.cpp:34-57)
// All are grid-stride, 16-byte vectorised and coalesced; grids are sized from the SM count.
#pragma once

#include <type_traits>

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ib200 {

// cudaError_t of the most recent failing CUDA call on this host thread (what ib200_last_cuda_error returns).
inline thread_local int g_last_cuda_error = 0;
inline bool cuda_ok(cudaError_t e) {
    if (e == cudaSuccess) return true;
    g_last_cuda_error = static_cast<int>(e);
    (void)cudaGetLastError();
    return false;
}
constexpr int kErrCuda = 5;      // IB200_ERR_CUDA
inline int launch_status() { return cuda_ok(cudaGetLastError()) ? 0 : kErrCuda; }

// Where the rows of a [B, H, T, D] operand live: element strides of the batch, head and token axes
// (the D elements of a row are contiguous).  Dense row-major is {H*T*D, T*D, D}; a q/k/v slice of a packed
// [B, T, 3, H, D] projection is {T*3*H*D, D, 3*H*D}.
struct RowLayout {
    long sb, sh, st;
    int H;
    __host__ __device__ long row(long head, int t) const { return (head / H) * sb + (head % H) * sh + static_cast<long>(t) * st; }
};
inline RowLayout dense_layout(int H, int T, int D) { return RowLayout{static_cast<long>(H) * T * D, static_cast<long>(T) * D, D, H}; }

constexpr int kAuxThreads = 256;
constexpr int kAuxBlocks = 148 * 8;

// hi = bf16(x), lo = bf16(x - hi): 8 elements per thread, two 16-byte loads, two 16-byte stores.
// Reads rows through the operand's layout (any layout) and writes hi / lo dense, so the main kernels always see dense
// operand copies in fp32-I/O mode.  One launch splits every operand of a pass (q, k, v forward; q, k, v, dO backward):
// grid z selects the operand, grid y the head.
struct SplitJob {
    const float* in[4];
    uint4* hi[4];
    uint4* lo[4];
    RowLayout lin[4];
};
__device__ __forceinline__ void split_bf16_block(const SplitJob& job, int z, int T, int D) {
    const float* __restrict__ in = job.in[z];
    const RowLayout lin = job.lin[z];
    const int cpr = D / 8;                                   // 8-element chunks per row
    const long head = blockIdx.y;                            // one head per grid row
    const long base_in = lin.row(head, 0);
    const int n8 = T * cpr;
    uint4* __restrict__ hi_h = job.hi[z] + head * static_cast<long>(n8);
    uint4* __restrict__ lo_h = job.lo[z] + head * static_cast<long>(n8);
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += gridDim.x * blockDim.x) {
        const int t = i / cpr, c8 = i - t * cpr;
        const float4* src = reinterpret_cast<const float4*>(in + base_in + static_cast<long>(t) * lin.st + c8 * 8);
        const float4 a = src[0], b = src[1];
        const float x[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        uint32_t h[4], l[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const __nv_bfloat162 hh = __floats2bfloat162_rn(x[2 * e], x[2 * e + 1]);
            const float2 hf = __bfloat1622float2(hh);
            const __nv_bfloat162 ll = __floats2bfloat162_rn(x[2 * e] - hf.x, x[2 * e + 1] - hf.y);
            h[e] = *reinterpret_cast<const uint32_t*>(&hh);
            l[e] = *reinterpret_cast<const uint32_t*>(&ll);
        }
        hi_h[i] = make_uint4(h[0], h[1], h[2], h[3]);
        lo_h[i] = make_uint4(l[0], l[1], l[2], l[3]);
    }
}

// Workspace header (see attn_api.cu): word 0 = sticky device status, word 1 = draw counter of the persistent kernels
// (zero at every launch), word 3 = "status word is valid" mark for a workspace that arrives uninitialised.
constexpr int kHeaderMagic = 0x1b200a77;
__device__ __forceinline__ void prepare_header(int* hdr) {
    if (hdr[3] != kHeaderMagic) { hdr[0] = 0; hdr[3] = kHeaderMagic; }
    hdr[1] = 0;
}

// Forward pre-pass of the fp32-I/O path: q, k, v -> hi / lo copies (grid z = operand), and the header.
__global__ void __launch_bounds__(kAuxThreads) split_bf16_kernel(SplitJob job, int* header, int T, int D) {
    if (header && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && threadIdx.x == 0) prepare_header(header);
    split_bf16_block(job, blockIdx.z, T, D);
}

// n_ops operands (3 or 4) in one launch.
inline int launch_split_bf16(const SplitJob& job, int n_ops, int* header, long heads, int T, int D, cudaStream_t stream) {
    const int n8 = T * (D / 8);
    int bx = (n8 + kAuxThreads - 1) / kAuxThreads;
    if (bx > 64) bx = 64;                                    // grid-stride inside a head beyond that
    dim3 grid(bx, static_cast<unsigned>(heads), static_cast<unsigned>(n_ops));
    split_bf16_kernel<<<grid, kAuxThreads, 0, stream>>>(job, header, T, D);
    return launch_status();
}

// Dense casts between fp32 and bf16 (round to nearest even), 8 elements per thread: for callers whose tensors are
// fp32 (the reference has no 16-bit DType, include/inferno/core/dtype.h:17-26) but who run the bf16 kernels.
__global__ void __launch_bounds__(kAuxThreads) cast_f32_bf16_kernel(const float4* __restrict__ in, uint4* __restrict__ out, long n8) {
    for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n8; i += static_cast<long>(gridDim.x) * blockDim.x) {
        const float4 a = in[2 * i], b = in[2 * i + 1];
        const __nv_bfloat162 p0 = __floats2bfloat162_rn(a.x, a.y), p1 = __floats2bfloat162_rn(a.z, a.w);
        const __nv_bfloat162 p2 = __floats2bfloat162_rn(b.x, b.y), p3 = __floats2bfloat162_rn(b.z, b.w);
        out[i] = make_uint4(*reinterpret_cast<const uint32_t*>(&p0), *reinterpret_cast<const uint32_t*>(&p1),
                            *reinterpret_cast<const uint32_t*>(&p2), *reinterpret_cast<const uint32_t*>(&p3));
    }
}

__global__ void __launch_bounds__(kAuxThreads) cast_bf16_f32_kernel(const uint4* __restrict__ in, float4* __restrict__ out, long n8) {
    for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n8; i += static_cast<long>(gridDim.x) * blockDim.x) {
        const uint4 v = in[i];
        out[2 * i] = make_float4(__uint_as_float(v.x << 16), __uint_as_float(v.x & 0xffff0000u), __uint_as_float(v.y << 16), __uint_as_float(v.y & 0xffff0000u));
        out[2 * i + 1] = make_float4(__uint_as_float(v.z << 16), __uint_as_float(v.z & 0xffff0000u), __uint_as_float(v.w << 16), __uint_as_float(v.w & 0xffff0000u));
    }
}

// One row of D elements is covered by TPR threads, each loading 16 bytes of O and of dO.
// Outputs are laid out [heads, T_pad] with T_pad a multiple of 64 so that the backward kernel can
// fetch the 64 values of a query block with one aligned bulk copy; both are stored negated and
// pre-scaled the way that kernel consumes them:
//   ndelta[h, t] = -sum_d O[h,t,d] * dO[h,t,d]        nlse2[h, t] = -lse[h,t] * log2(e)
// Padding rows (t >= T) are written as 0.
template <int D, bool F32>
__device__ __forceinline__ void delta_block(const void* __restrict__ o_, const void* __restrict__ do_, const float* __restrict__ lse,
                                            float* __restrict__ ndelta, float* __restrict__ nlse2, const RowLayout& lo, const RowLayout& ldo,
                                            int T, int T_pad) {
    constexpr int EPT = F32 ? 4 : 8;              // elements per 16-byte load
    constexpr int TPR = D / EPT;                  // threads per row (8 or 16)
    constexpr int RPB = kAuxThreads / TPR;        // rows per block per step
    constexpr int U = 4;                          // steps per block: 2 * U independent 16-byte loads in flight per thread
    using Vec = typename std::conditional<F32, float4, uint4>::type;
    const int sub = threadIdx.x % TPR;
    const long head = blockIdx.y;                 // one head per grid row: no per-row divisions
    const int t0 = blockIdx.x * (RPB * U) + threadIdx.x / TPR;
    const long base_o = lo.row(head, 0), base_do = ldo.row(head, 0);
    Vec a[U], b[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int t = t0 + u * RPB;
        if (t < T) {
            if constexpr (F32) {
                a[u] = reinterpret_cast<const float4*>(static_cast<const float*>(o_) + base_o + static_cast<long>(t) * lo.st)[sub];
                b[u] = reinterpret_cast<const float4*>(static_cast<const float*>(do_) + base_do + static_cast<long>(t) * ldo.st)[sub];
            } else {
                a[u] = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(o_) + base_o + static_cast<long>(t) * lo.st)[sub];
                b[u] = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(do_) + base_do + static_cast<long>(t) * ldo.st)[sub];
            }
        }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int t = t0 + u * RPB;
        const bool live = t < T;
        float acc = 0.f;
        if (live) {
            if constexpr (F32) {
                acc = a[u].x * b[u].x + a[u].y * b[u].y + a[u].z * b[u].z + a[u].w * b[u].w;
            } else {
                const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a[u]);
                const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&b[u]);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 fa = __bfloat1622float2(pa[e]), fb = __bfloat1622float2(pb[e]);
                    acc = fmaf(fa.x, fb.x, acc);
                    acc = fmaf(fa.y, fb.y, acc);
                }
            }
        }
        // every thread of a row group takes part in the shuffles (t is uniform per group)
#pragma unroll
        for (int off = TPR / 2; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
        if (sub == 0 && t < T_pad) {
            const long prow = head * T_pad + t;
            ndelta[prow] = -acc;
            nlse2[prow] = live ? lse[head * T + t] * -1.4426950408889634f : 0.f;
        }
    }
}

// The backward's one pre-pass launch.  Grid y = head; grid z selects the job:
//   z = 0      -delta and -lse*log2e of the head's rows (delta_block), and the workspace header
//   z = 1      zeroes the head's slice of the fp32 dQ accumulator (the main kernel adds into it)
//   z = 2..5   (fp32 I/O only) q, k, v, dO -> hi / lo bf16 copies
// grid x = blocks of 64 rows, which is what delta_block needs; the other jobs stride over it.
struct BwdPrepassJob {
    const void* o;
    const void* dO;
    const float* lse;
    float* ndelta;
    float* nlse2;
    RowLayout lo, ldo;
    float4* dq_acc;        // dense [heads, T, D] fp32
    int* header;
    SplitJob split;        // used when F32
};
template <int D, bool F32>
__global__ void __launch_bounds__(kAuxThreads) bwd_prepass_kernel(BwdPrepassJob job, int T, int T_pad) {
    const int z = blockIdx.z;
    if (z == 0) {
        if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) prepare_header(job.header);
        delta_block<D, F32>(job.o, job.dO, job.lse, job.ndelta, job.nlse2, job.lo, job.ldo, T, T_pad);
    } else if (z == 1) {
        const long n4 = static_cast<long>(T) * (D / 4);                      // float4 chunks of this head's accumulator slice
        float4* dst = job.dq_acc + static_cast<long>(blockIdx.y) * n4;
        for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n4; i += static_cast<long>(gridDim.x) * blockDim.x)
            dst[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    } else if constexpr (F32) {
        split_bf16_block(job.split, z - 2, T, D);
    }
}

template <int D, bool F32>
inline int launch_bwd_prepass(const BwdPrepassJob& job, long heads, int T, int T_pad, cudaStream_t stream) {
    constexpr int RPB = kAuxThreads / (D / (F32 ? 4 : 8));
    dim3 grid((T_pad + RPB * 4 - 1) / (RPB * 4), static_cast<unsigned>(heads), F32 ? 6 : 2);
    bwd_prepass_kernel<D, F32><<<grid, kAuxThreads, 0, stream>>>(job, T, T_pad);
    return launch_status();
}

// out[row, :] = scale * acc[row, :], 8 elements per thread; acc is dense [heads, T, D], out follows `lout`.
// One head per grid row and a power-of-two row length: no divisions in the index arithmetic; U chunks per thread
// so that 2 * U 16-byte loads are in flight.
template <int D, bool F32>
__global__ void __launch_bounds__(kAuxThreads) dq_finish_kernel(const float4* __restrict__ acc, void* __restrict__ out, float scale,
                                                                RowLayout lout, int T) {
    constexpr int CPR = D / 8;                    // 8-element chunks per row
    constexpr int U = 4;
    const long head = blockIdx.y;
    const long base_out = lout.row(head, 0);
    const float4* acc_h = acc + head * static_cast<long>(T) * CPR * 2;
    const int n8 = T * CPR;                       // chunks of this head
    const int i0 = blockIdx.x * (kAuxThreads * U) + threadIdx.x;
    float4 a[U], b[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int i = i0 + u * kAuxThreads;
        if (i < n8) { a[u] = acc_h[2 * i]; b[u] = acc_h[2 * i + 1]; }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int i = i0 + u * kAuxThreads;
        if (i >= n8) continue;
        const int t = i / CPR, c8 = i % CPR;
        const long dst = base_out + static_cast<long>(t) * lout.st + c8 * 8;
        float4 x = a[u], y = b[u];
        x.x *= scale; x.y *= scale; x.z *= scale; x.w *= scale;
        y.x *= scale; y.y *= scale; y.z *= scale; y.w *= scale;
        if constexpr (F32) {
            float4* o4 = reinterpret_cast<float4*>(static_cast<float*>(out) + dst);
            o4[0] = x;
            o4[1] = y;
        } else {
            uint4 v;
            __nv_bfloat162 t2;
            t2 = __floats2bfloat162_rn(x.x, x.y); v.x = *reinterpret_cast<uint32_t*>(&t2);
            t2 = __floats2bfloat162_rn(x.z, x.w); v.y = *reinterpret_cast<uint32_t*>(&t2);
            t2 = __floats2bfloat162_rn(y.x, y.y); v.z = *reinterpret_cast<uint32_t*>(&t2);
            t2 = __floats2bfloat162_rn(y.z, y.w); v.w = *reinterpret_cast<uint32_t*>(&t2);
            *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(out) + dst) = v;
        }
    }
}

template <int D, bool F32>
inline int launch_dq_finish(const float* acc, void* out, float scale, const RowLayout& lout, long heads, int T, cudaStream_t stream) {
    const int n8 = T * (D / 8);
    dim3 grid((n8 + kAuxThreads * 4 - 1) / (kAuxThreads * 4), static_cast<unsigned>(heads), 1);
    dq_finish_kernel<D, F32><<<grid, kAuxThreads, 0, stream>>>(reinterpret_cast<const float4*>(acc), out, scale, lout, T);
    return launch_status();
}

}  // namespace ib200
