// C ABI of the attention kernels (declared in include/inferno_b200_attn.h).
// Host side only: argument checks, tensor maps, workspace carving and launches.
#include "../../include/inferno_b200_attn.h"

#include <cuda.h>
#include <cuda_runtime.h>
#include <math.h>

#include <atomic>

#include "attn_aux.cuh"
#include "attn_bwd.cuh"
#include "attn_bwd_persist.cuh"
#include "attn_fwd.cuh"
#include "attn_fwd_persist.cuh"
#include "linear_gemm.cuh"

namespace {

using namespace ib200;

thread_local cudaEvent_t g_ev[4] = {nullptr, nullptr, nullptr, nullptr};   // fwd start/stop, bwd start/stop

// Timing events are an observability aid: a handle that has gone stale (the hook is per host thread and a
// caller may have destroyed its events without switching the hook off on that thread) must not fail the launch.
inline void record_timing_event(int which, cudaStream_t stream) {
    if (g_ev[which] && cudaEventRecord(g_ev[which], stream) != cudaSuccess) {
        (void)cudaGetLastError();
        g_ev[which] = nullptr;
    }
}

// Checked build: the extents the device-side range checks compare against, set on `stream` ahead of every main kernel
// (a debugging aid: launches on different streams share the one constant and must not overlap).
#ifdef IB200_BOUNDS
int set_bounds(int d0, int d1, int d2, int d3, int rows3, int relaxed, unsigned tmem_cols, int* status, cudaStream_t stream) {
    const BoundsInfo b{{d0, d1, d2, d3}, rows3, relaxed, tmem_cols, status};
    return cuda_ok(cudaMemcpyToSymbolAsync(c_bounds, &b, sizeof(b), 0, cudaMemcpyHostToDevice, stream)) ? IB200_OK : IB200_ERR_CUDA;
}
#define IB200_SET_BOUNDS(...) do { if (int rc_ = set_bounds(__VA_ARGS__)) return rc_; } while (0)
#else
#define IB200_SET_BOUNDS(...) do {} while (0)
#endif

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) p = nullptr;
        (void)cudaGetLastError();
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// Tensor map over a [B, H, T, D] operand with arbitrary batch / head / token strides, seen as the 4-D tensor
// {D, T, H, B}; box = [box_rows x 128 bytes], 128B swizzle.  Rows past T are zero-filled on load and clipped
// on store; a tile never crosses into another head.
bool make_tmap(CUtensorMap* m, const void* base, bool f32, int D, int T, const RowLayout& L, long BH, int box_rows) {
    EncodeTiledFn enc = encode_fn();
    if (!enc) return false;
    const cuuint64_t es = f32 ? 4 : 2;
    const long B = BH / L.H;
    cuuint64_t dims[4] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(T), static_cast<cuuint64_t>(L.H), static_cast<cuuint64_t>(B)};
    cuuint64_t strides[3] = {static_cast<cuuint64_t>(L.st) * es, static_cast<cuuint64_t>(L.sh) * es, static_cast<cuuint64_t>(L.sb) * es};
    cuuint32_t box[4] = {static_cast<cuuint32_t>(128 / es), static_cast<cuuint32_t>(box_rows), 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = enc(m, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4,
                     const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

// Tensor map over a row-major bf16 matrix [rows, cols]; box = [box_rows x 64 columns], 128B swizzle.
bool make_tmap_2d(CUtensorMap* m, const void* base, long rows, long cols, int box_rows) {
    EncodeTiledFn enc = encode_fn();
    if (!enc) return false;
    cuuint64_t dims[3] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows), 1};
    cuuint64_t strides[2] = {static_cast<cuuint64_t>(cols) * 2, static_cast<cuuint64_t>(rows) * static_cast<cuuint64_t>(cols) * 2};
    cuuint32_t box[3] = {64, static_cast<cuuint32_t>(box_rows), 1};
    cuuint32_t estr[3] = {1, 1, 1};
    return enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline size_t round_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

constexpr size_t kHeaderBytes = 256;

// Workspace header: word 0 = device status (sticky: the first expired wait stays recorded until ib200_attn_check
// has read it), word 1 = draw counter of the persistent kernels (zero at every launch), word 3 = "status word is
// valid" mark.  A workspace arrives uninitialised, so the mark decides whether word 0 is a status or garbage.
__global__ void prepare_header_kernel(int* hdr) {
    if (threadIdx.x == 0) prepare_header(hdr);
}
int prepare_header(void* ws, cudaStream_t stream) {
    prepare_header_kernel<<<1, 32, 0, stream>>>(static_cast<int*>(ws));
    return launch_status();
}

struct Problem {
    long BH, N;        // heads, elements per tensor
    bool f32;
};

int check_common(int B, int H, int T, int D, int dtype, int math_mode, int causal) {
    if (B <= 0 || H <= 0 || T <= 0 || D <= 0) return IB200_ERR_INVALID_ARGUMENT;
    if (dtype != IB200_DTYPE_F32 && dtype != IB200_DTYPE_BF16) return IB200_ERR_INVALID_ARGUMENT;
    if (causal != 0 && causal != 1) return IB200_ERR_INVALID_ARGUMENT;
    if (dtype == IB200_DTYPE_F32 && math_mode != IB200_MATH_SPLIT_BF16) return IB200_ERR_UNSUPPORTED;
    if (dtype == IB200_DTYPE_BF16 && D != 64 && D != 128) return IB200_ERR_UNSUPPORTED;
    if (dtype == IB200_DTYPE_F32 && D != 64) return IB200_ERR_UNSUPPORTED;
    // one head per grid row of the helper kernels and of the one-CTA-per-item main kernels
    if (static_cast<long>(B) * H > 65535L) return IB200_ERR_UNSUPPORTED;
    return IB200_OK;
}

size_t fwd_ws_bytes(long N, bool f32) { return kHeaderBytes + (f32 ? 6 * round_up(N * 2, 256) : 0); }
inline int pad64(int T) { return (T + 63) / 64 * 64; }
size_t bwd_ws_bytes(long N, long BH, int T, bool f32) {
    return kHeaderBytes + round_up(N * 4, 256) /*dq accumulator*/ + 2 * round_up(static_cast<size_t>(BH) * pad64(T) * 4, 256) /*-delta, -lse*log2e*/ +
           (f32 ? 8 * round_up(N * 2, 256) : 0);
}

int device_ok() {
    int dev = 0;
    if (!cuda_ok(cudaGetDevice(&dev))) return IB200_ERR_NO_DEVICE;
    int major = 0;
    if (!cuda_ok(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev))) return IB200_ERR_NO_DEVICE;
    return major == 10 ? IB200_OK : IB200_ERR_NO_DEVICE;
}

// Number of head groups of a persistent kernel's item list (see locate_item).  The CTAs draw items in list order, so at
// any time they work on a window of about one round (one item per CTA) of the list.  With every head in one group the window
// would span up to one head per CTA, and the tiles the CTAs of a head share (K / V in the forward; Q / dO and the dQ
// accumulator in the backward: `shared_bytes_per_head`) would fall out of L2.  So a group is as many heads as keep those
// tiles within 48 MB, but never fewer than two rounds of items: a group starts with its heaviest items, and it is the
// second round's light items that let the drawing even out the CTAs before the list ends.
int persist_head_groups(int ctas, int items_per_head, long BH, size_t shared_bytes_per_head) {
    const long items = static_cast<long>(items_per_head) * BH;
    long g = static_cast<long>((48u << 20) / (shared_bytes_per_head ? shared_bytes_per_head : 1));
    if (g < 1) g = 1;
    long n_groups = (BH + g - 1) / g;
    if (n_groups > items / (2L * ctas)) n_groups = items / (2L * ctas);
    return static_cast<int>(n_groups < 1 ? 1 : n_groups);
}

// Persistent CTAs walking (head, query-tile pair) items, heaviest first.  SPLIT: fp32 I/O, operands given as dense
// (hi, lo) bf16 copies (q_lo, k_lo, v_lo), output fp32.
template <int D, bool SPLIT>
int launch_fwd_persist(const void* q, const void* q_lo, const void* k, const void* k_lo, const void* v, const void* v_lo, void* o,
                       const RowLayout& lq, const RowLayout& lk, const RowLayout& lv, const RowLayout& lo, float* lse, int* status,
                       long BH, int T, float scale, int causal, cudaStream_t stream) {
    using TR = FwdPersistTraits<D, SPLIT>;
    CUtensorMap tq, tql, tk, tkl, tv, tvl, to;
    if (!make_tmap(&tq, q, false, D, T, lq, BH, 128) || !make_tmap(&tk, k, false, D, T, lk, BH, 128) ||
        !make_tmap(&tv, v, false, D, T, lv, BH, 128) || !make_tmap(&to, o, SPLIT, D, T, lo, BH, 128))
        return IB200_ERR_CUDA;
    if (SPLIT) {
        if (!make_tmap(&tql, q_lo, false, D, T, lq, BH, 128) || !make_tmap(&tkl, k_lo, false, D, T, lk, BH, 128) ||
            !make_tmap(&tvl, v_lo, false, D, T, lv, BH, 128))
            return IB200_ERR_CUDA;
    } else {
        tql = tq; tkl = tk; tvl = tv;
    }
    if (!cuda_ok(cudaFuncSetAttribute(attn_fwd_persist_kernel<TR>, cudaFuncAttributeMaxDynamicSharedMemorySize, TR::SMEM_BYTES)))
        return IB200_ERR_CUDA;
    FwdPersistParams pp;
    pp.p.lse = lse;
    pp.p.status = status;
    pp.p.T = T;
    pp.p.BH = static_cast<int>(BH);
    pp.p.H = lq.H;
    pp.p.causal = causal;
    pp.p.scale_log2 = scale * 1.4426950408889634f;
    pp.pairs_per_head = (T + 255) / 256;
    const long items = static_cast<long>(pp.pairs_per_head) * BH;
    if (items > 0x7fffffffL) return IB200_ERR_UNSUPPORTED;
    pp.n_items = static_cast<int>(items);
    int dev = 0, sms = 148;
    if (cuda_ok(cudaGetDevice(&dev))) (void)cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int grid = static_cast<int>(items < sms ? items : sms);
    pp.n_groups = persist_head_groups(sms, pp.pairs_per_head, BH, static_cast<size_t>(T) * D * (SPLIT ? 8 : 4) /*K, V*/);
    pp.next_item = status + 1;              // second word of the workspace header, zeroed before every launch
    IB200_SET_BOUNDS(D, T, lq.H, static_cast<int>(BH / lq.H), static_cast<int>(BH), 0, TR::TM_COLS, status, stream);
    record_timing_event(0, stream);
    attn_fwd_persist_kernel<TR><<<grid, TR::THREADS, TR::SMEM_BYTES, stream>>>(tq, tql, tk, tkl, tv, tvl, to, pp);
    const bool launched = cuda_ok(cudaGetLastError());
    record_timing_event(1, stream);
    return launched ? IB200_OK : IB200_ERR_CUDA;
}

// Persistent CTAs walking (head, key tile) items, longest walks first.  SPLIT (fp32 I/O): every operand is given as dense
// (hi, lo) bf16 copies, index 0 / 1 of the pointer pairs; dK / dV come out as fp32.
template <class TR>
int launch_bwd_persist(const void* const q[2], const void* const k[2], const void* const v[2], const void* const dO[2],
                       const RowLayout& lq, const RowLayout& lk, const RowLayout& lv, const RowLayout& ldo, const RowLayout& ldk,
                       const RowLayout& ldv, const float* nlse2, const float* ndelta, int T_pad, float* dq_acc, float dq_scale, void* dk, void* dv,
                       int* status, long BH, int T, float scale, int causal, cudaStream_t stream) {
    CUtensorMap tq[2], tk[2], tv[2], tdo[2], tdk, tdv, tdq;
    for (int i = 0; i < (TR::SPLIT ? 2 : 1); ++i) {
        if (!make_tmap(&tq[i], q[i], false, TR::D, T, lq, BH, TR::BQ) || !make_tmap(&tdo[i], dO[i], false, TR::D, T, ldo, BH, TR::BQ) ||
            !make_tmap(&tk[i], k[i], false, TR::D, T, lk, BH, TR::BKV) || !make_tmap(&tv[i], v[i], false, TR::D, T, lv, BH, TR::BKV))
            return IB200_ERR_CUDA;
    }
    if (!TR::SPLIT) { tq[1] = tq[0]; tk[1] = tk[0]; tv[1] = tv[0]; tdo[1] = tdo[0]; }
    if (!make_tmap(&tdk, dk, TR::SPLIT, TR::D, T, ldk, BH, TR::BKV) || !make_tmap(&tdv, dv, TR::SPLIT, TR::D, T, ldv, BH, TR::BKV))
        return IB200_ERR_CUDA;
    {
        // fp32 dQ accumulator, whole rows of D floats per box row, no swizzle (the staging tile is plain row-major)
        EncodeTiledFn enc = encode_fn();
        if (!enc) return IB200_ERR_CUDA;
        cuuint64_t dims[3] = {static_cast<cuuint64_t>(TR::D), static_cast<cuuint64_t>(T), static_cast<cuuint64_t>(BH)};
        cuuint64_t strides[2] = {static_cast<cuuint64_t>(TR::D) * 4, static_cast<cuuint64_t>(T) * TR::D * 4};
        cuuint32_t box[3] = {static_cast<cuuint32_t>(TR::D), static_cast<cuuint32_t>(TR::BQ), 1};
        cuuint32_t estr[3] = {1, 1, 1};
        if (enc(&tdq, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, dq_acc, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return IB200_ERR_CUDA;
    }
    if (!cuda_ok(cudaFuncSetAttribute(attn_bwd_persist_kernel<TR>, cudaFuncAttributeMaxDynamicSharedMemorySize, TR::SMEM_BYTES)))
        return IB200_ERR_CUDA;
    BwdParams prm;
    prm.nlse2 = nlse2;
    prm.ndelta = ndelta;
    prm.T_pad = T_pad;
    prm.status = status;
    prm.T = T;
    prm.BH = static_cast<int>(BH);
    prm.H = lq.H;
    prm.causal = causal;
    prm.scale = scale;
    prm.scale_log2 = scale * 1.4426950408889634f;
    prm.dq_scale = dq_scale;
    const long items = static_cast<long>((T + TR::BKV - 1) / TR::BKV) * BH;
    if (items > 0x7fffffffL) return IB200_ERR_UNSUPPORTED;
    int dev = 0, sms = 148;
    if (cuda_ok(cudaGetDevice(&dev))) (void)cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int grid = static_cast<int>(items < sms ? items : sms);
    const int n_groups = persist_head_groups(sms, (T + TR::BKV - 1) / TR::BKV, BH,
                                             static_cast<size_t>(T) * TR::D * (TR::SPLIT ? 12 : 8) /*Q, dO (hi + lo), fp32 dQ*/);
    IB200_SET_BOUNDS(TR::D, T, lq.H, static_cast<int>(BH / lq.H), static_cast<int>(BH), 0, TR::TM_COLS, status, stream);
    record_timing_event(2, stream);
    attn_bwd_persist_kernel<TR><<<grid, TR::THREADS, TR::SMEM_BYTES, stream>>>(tq[0], tq[1], tk[0], tk[1], tv[0], tv[1], tdo[0], tdo[1], tdk, tdv, tdq, prm,
                                                                               static_cast<int>(items), n_groups,
                                                                               status + 1 /*draw counter: header word zeroed before every launch*/);
    const bool launched = cuda_ok(cudaGetLastError());
    record_timing_event(3, stream);
    return launched ? IB200_OK : IB200_ERR_CUDA;
}

struct BwdLayouts {
    RowLayout q, k, v, o, dO, dq, dk, dv;
};

// pre-pass (delta, accumulator zeroing, header, fp32 operand splits) -> main kernel -> dQ finish.
// Workspace: [header | dq accumulator | -delta, -lse*log2e | (fp32 only) dense hi/lo bf16 copies of q, k, v, dO].
template <int D, bool F32>
int launch_bwd_typed(const void* q, const void* k, const void* v, const void* o, const void* dO, const float* lse,
                     void* dq, void* dk, void* dv, const BwdLayouts& L, long BH, int T, float scale, int causal,
                     uint8_t* ws, cudaStream_t stream) {
    const long N = BH * T * D;
    int* status = reinterpret_cast<int*>(ws);
    float* dq_acc = reinterpret_cast<float*>(ws + kHeaderBytes);
    // fp32 I/O with a dense dQ: the partial tiles, scaled, are added straight into the caller's dQ (zeroed by the pre-pass),
    // and no finish pass runs; otherwise they meet in the workspace's fp32 accumulator, which dq_finish_kernel scales and casts
    const RowLayout dense = dense_layout(L.q.H, T, D);
    const bool dq_direct = F32 && L.dq.sb == dense.sb && L.dq.sh == dense.sh && L.dq.st == dense.st;
    if (dq_direct) dq_acc = static_cast<float*>(dq);
    uint8_t* after_acc = ws + kHeaderBytes + round_up(N * 4, 256);
    const int T_pad = pad64(T);
    const size_t vec_bytes = round_up(static_cast<size_t>(BH) * T_pad * 4, 256);
    float* ndelta = reinterpret_cast<float*>(after_acc);
    float* nlse2 = reinterpret_cast<float*>(after_acc + vec_bytes);
    BwdPrepassJob job;
    job.o = o; job.dO = dO; job.lse = lse; job.ndelta = ndelta; job.nlse2 = nlse2;
    job.lo = L.o; job.ldo = L.dO;
    job.dq_acc = reinterpret_cast<float4*>(dq_acc);
    job.header = status;
    const void* qp[2] = {q, q}; const void* kp[2] = {k, k}; const void* vp[2] = {v, v}; const void* dop[2] = {dO, dO};
    RowLayout lq = L.q, lk = L.k, lv = L.v, ldo = L.dO;
    if (F32) {
        uint8_t* base = after_acc + 2 * vec_bytes;
        const size_t slab = round_up(N * 2, 256);
        const void** dst[4] = {qp, kp, vp, dop};
        const float* src[4] = {static_cast<const float*>(q), static_cast<const float*>(k), static_cast<const float*>(v), static_cast<const float*>(dO)};
        const RowLayout* lsrc[4] = {&L.q, &L.k, &L.v, &L.dO};
        for (int i = 0; i < 4; ++i) {
            job.split.in[i] = src[i];
            job.split.hi[i] = reinterpret_cast<uint4*>(base + (2 * i) * slab);
            job.split.lo[i] = reinterpret_cast<uint4*>(base + (2 * i + 1) * slab);
            job.split.lin[i] = *lsrc[i];
            dst[i][0] = job.split.hi[i];
            dst[i][1] = job.split.lo[i];
        }
        lq = lk = lv = ldo = dense_layout(L.q.H, T, D);      // the hi/lo copies are dense
    } else {
        for (int i = 0; i < 4; ++i) { job.split.in[i] = nullptr; job.split.hi[i] = job.split.lo[i] = nullptr; job.split.lin[i] = L.q; }
    }
    int rc = launch_bwd_prepass<D, F32>(job, BH, T, T_pad, stream);
    if (rc) return rc;
    rc = launch_bwd_persist<BwdTraits<D, F32>>(qp, kp, vp, dop, lq, lk, lv, ldo, L.dk, L.dv, nlse2, ndelta, T_pad, dq_acc,
                                               dq_direct ? scale : 1.f, dk, dv, status, BH, T, scale, causal, stream);
    if (rc || dq_direct) return rc;
    return launch_dq_finish<D, F32>(dq_acc, dq, scale, L.dq, BH, T, stream);
}

int launch_bwd_all(const void* q, const void* k, const void* v, const void* o, const void* dO, const float* lse,
                   void* dq, void* dk, void* dv, const BwdLayouts& L, long BH, int T, int D, float scale, int causal, bool f32,
                   uint8_t* ws, cudaStream_t stream) {
    if (f32) return launch_bwd_typed<64, true>(q, k, v, o, dO, lse, dq, dk, dv, L, BH, T, scale, causal, ws, stream);
    if (D == 64) return launch_bwd_typed<64, false>(q, k, v, o, dO, lse, dq, dk, dv, L, BH, T, scale, causal, ws, stream);
    return launch_bwd_typed<128, false>(q, k, v, o, dO, lse, dq, dk, dv, L, BH, T, scale, causal, ws, stream);
}

// A caller-supplied layout (NULL = dense), checked: rows of D elements must start on 16-byte boundaries.
int resolve_layout(const ib200_layout* in, int H, int T, int D, bool f32, RowLayout* out) {
    if (!in) { *out = dense_layout(H, T, D); return IB200_OK; }
    const long unit = f32 ? 4 : 8;      // elements per 16 bytes
    if (in->stride_b <= 0 || in->stride_h <= 0 || in->stride_t <= 0) return IB200_ERR_INVALID_ARGUMENT;
    if (in->stride_b % unit || in->stride_h % unit || in->stride_t % unit) return IB200_ERR_MISALIGNED;
    if (in->stride_t < D || in->stride_h < D) return IB200_ERR_INVALID_ARGUMENT;
    *out = RowLayout{static_cast<long>(in->stride_b), static_cast<long>(in->stride_h), static_cast<long>(in->stride_t), H};
    return IB200_OK;
}

// Scratch for ib200_attn_bwd_static.  In host code this name is only a handle for the runtime; the
// device address is looked up once per device with cudaGetSymbolAddress and that pointer is what
// the launch path receives.
static __device__ __align__(256) unsigned char g_static_scratch[IB200_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
// Filled on first use per device.  Two host threads that race on the first call both look the address up and both
// store the same value, so a relaxed atomic is all the cache needs.
std::atomic<void*> g_static_scratch_addr[kMaxDevices];

// Device address of the static scratch on the current device (set-up on first use per device).
int static_scratch(void** out) {
    int dev = 0;
    if (!cuda_ok(cudaGetDevice(&dev))) return IB200_ERR_NO_DEVICE;
    if (dev < 0 || dev >= kMaxDevices) return IB200_ERR_UNSUPPORTED;
    void* p = g_static_scratch_addr[dev].load(std::memory_order_relaxed);
    if (!p) {
        if (!cuda_ok(cudaGetSymbolAddress(&p, g_static_scratch)) || !p) return IB200_ERR_CUDA;
        g_static_scratch_addr[dev].store(p, std::memory_order_relaxed);
    }
    *out = p;
    return IB200_OK;
}

// Self-test of the bounded-wait path, without any fault: one CTA allocates TMEM, warp 1 waits on an mbarrier that
// nothing ever arrives on and gives up after `limit_ns`, warp 2 waits on the same barrier with the product limit and
// must come back as soon as warp 1 has raised the CTA's abort flag; the CTA then frees its TMEM and exits normally.
__global__ void __launch_bounds__(128, 1) wait_expiry_probe_kernel(int* status, unsigned long long limit_ns) {
    __shared__ uint64_t bar;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    const int warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) { abort_flag = 0; mbar_init(&bar, 1); fence_mbar_init(); }
    if (warp == 0) { tmem_alloc(&tmem_slot, 32); tmem_relinquish(); }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    AbortCtx ab{&abort_flag, status};
    if (warp == 1) mbar_wait_limit(&bar, 0, ab, 90, limit_ns);
    if (warp == 2) mbar_wait(&bar, 0, ab, 91);
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_slot, 32);
}

bool header_is_builtin(const void* header) {
    for (int d = 0; d < kMaxDevices; ++d)
        if (header && g_static_scratch_addr[d].load(std::memory_order_relaxed) == header) return true;
    return false;
}

template <bool A_MN, bool B_MN>
int launch_gemm(const void* a, const void* b, void* c, const float* bias, int M, int N, int K, cudaStream_t stream) {
    using TR = GemmTraits;
    // a runtime call first: it makes the primary context current on this host thread (a framework's worker
    // thread may never have touched CUDA), which the driver's tensor-map encoder needs
    if (!cuda_ok(cudaFuncSetAttribute(gemm_bf16_kernel<A_MN, B_MN>, cudaFuncAttributeMaxDynamicSharedMemorySize, TR::SMEM_BYTES)))
        return IB200_ERR_CUDA;
    CUtensorMap ta, tb, tc;
    // A: [M,K] (box 128 rows) or stored [K,M] (box 64 k-rows); B: stored [K,N] (box 64 k-rows) or [N,K] (box 256 rows)
    const bool ok = (A_MN ? make_tmap_2d(&ta, a, K, M, 64) : make_tmap_2d(&ta, a, M, K, 128)) &&
                    (B_MN ? make_tmap_2d(&tb, b, K, N, 64) : make_tmap_2d(&tb, b, N, K, 256)) && make_tmap_2d(&tc, c, M, N, 128);
    if (!ok) return IB200_ERR_CUDA;
    int dev = 0, sms = 148;
    if (cuda_ok(cudaGetDevice(&dev))) (void)cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const long tiles = static_cast<long>((M + TR::BM - 1) / TR::BM) * ((N + TR::BN - 1) / TR::BN);
    // Split-K when the tiles would leave more than half of the SMs idle and K is long enough to cut: as many slabs as
    // fit in one wave, each at least eight 64-wide k-slices.  The slabs add into C, so C is zeroed first.
    const int k_slices = (K + TR::BK - 1) / TR::BK;
    int splits = 1;
    if (tiles * 2 <= sms) {
        splits = static_cast<int>(sms / tiles);
        if (splits > 8) splits = 8;
        while (splits > 1 && k_slices / splits < 8) --splits;
    }
    if (splits > 1 && !cuda_ok(cudaMemsetAsync(c, 0, static_cast<size_t>(M) * N * 2, stream))) return IB200_ERR_CUDA;
    GemmParams prm;
    prm.bias = bias;
    prm.M = M; prm.N = N; prm.K = K;
    prm.splits = splits;
    // an expired wait is recorded in the status word of the library's built-in buffer (read by ib200_attn_check_static)
    void* builtin = nullptr;
    prm.status = static_scratch(&builtin) == IB200_OK ? static_cast<int*>(builtin) : nullptr;
    const long units = tiles * splits;
    const int grid = static_cast<int>(units < sms ? units : sms);       // persistent: one CTA per SM
    IB200_SET_BOUNDS(0, 0, 0, 0, 0, 1, TR::TM_COLS, prm.status, stream);
    gemm_bf16_kernel<A_MN, B_MN><<<grid, TR::THREADS, TR::SMEM_BYTES, stream>>>(ta, tb, tc, prm);
    return cuda_ok(cudaGetLastError()) ? IB200_OK : IB200_ERR_CUDA;
}

int gemm_dispatch(const void* a, const void* b, void* c, const float* bias, int M, int N, int K, int a_t, int b_t, cudaStream_t stream) {
    if (!a || !b || !c) return IB200_ERR_INVALID_ARGUMENT;
    if (M <= 0 || N <= 0 || K <= 0 || (a_t != 0 && a_t != 1) || (b_t != 0 && b_t != 1)) return IB200_ERR_INVALID_ARGUMENT;
    if (M % 8 || N % 8 || K % 8) return IB200_ERR_UNSUPPORTED;
    if (!aligned16(a) || !aligned16(b) || !aligned16(c) || (bias && !aligned16(bias))) return IB200_ERR_MISALIGNED;
    int rc = device_ok();
    if (rc != IB200_OK) return rc;
    if (!a_t && !b_t) return launch_gemm<false, true>(a, b, c, bias, M, N, K, stream);
    if (!a_t && b_t) return launch_gemm<false, false>(a, b, c, bias, M, N, K, stream);
    if (a_t && !b_t) return launch_gemm<true, true>(a, b, c, bias, M, N, K, stream);
    return launch_gemm<true, false>(a, b, c, bias, M, N, K, stream);
}

int fwd_core(const void* q, const void* k, const void* v, void* o, float* lse, const ib200_layout* lq_, const ib200_layout* lk_,
             const ib200_layout* lv_, const ib200_layout* lo_, int B, int H, int T, int D, float scale, int causal, int dtype,
             int math_mode, void* workspace, size_t workspace_bytes, cudaStream_t stream) {
    if (!q || !k || !v || !o || !lse) return IB200_ERR_INVALID_ARGUMENT;
    int rc = check_common(B, H, T, D, dtype, math_mode, causal);
    if (rc != IB200_OK) return rc;
    if (!(scale > 0.f) || !isfinite(scale)) return IB200_ERR_INVALID_ARGUMENT;
    if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o) || !aligned16(lse)) return IB200_ERR_MISALIGNED;
    const long BH = static_cast<long>(B) * H;
    const long N = BH * T * D;
    const bool f32 = dtype == IB200_DTYPE_F32;
    RowLayout lq, lk, lv, lo;
    if ((rc = resolve_layout(lq_, H, T, D, f32, &lq)) || (rc = resolve_layout(lk_, H, T, D, f32, &lk)) ||
        (rc = resolve_layout(lv_, H, T, D, f32, &lv)) || (rc = resolve_layout(lo_, H, T, D, f32, &lo)))
        return rc;
    if (!workspace || !aligned16(workspace) || workspace_bytes < fwd_ws_bytes(N, f32)) return IB200_ERR_WORKSPACE;
    rc = device_ok();
    if (rc != IB200_OK) return rc;

    uint8_t* ws = static_cast<uint8_t*>(workspace);
    int* status = reinterpret_cast<int*>(ws);
    if (!f32 && (rc = prepare_header(ws, stream))) return rc;      // fp32 I/O: the split pre-pass prepares the header
    if (f32) {
        // fp32 operands are carried as dense (hi, lo) bf16 pairs
        const size_t slab = round_up(N * 2, 256);
        uint8_t* base = ws + kHeaderBytes;
        void* part[6];
        for (int i = 0; i < 6; ++i) part[i] = base + i * slab;
        SplitJob job;
        const float* src[3] = {static_cast<const float*>(q), static_cast<const float*>(k), static_cast<const float*>(v)};
        const RowLayout* lsrc[3] = {&lq, &lk, &lv};
        for (int i = 0; i < 3; ++i) {
            job.in[i] = src[i];
            job.hi[i] = static_cast<uint4*>(part[2 * i]);
            job.lo[i] = static_cast<uint4*>(part[2 * i + 1]);
            job.lin[i] = *lsrc[i];
        }
        job.in[3] = nullptr; job.hi[3] = job.lo[3] = nullptr; job.lin[3] = lq;
        rc = launch_split_bf16(job, 3, status, BH, T, D, stream);
        if (rc) return rc;
        const RowLayout dl = dense_layout(H, T, D);
        return launch_fwd_persist<64, true>(part[0], part[1], part[2], part[3], part[4], part[5], o, dl, dl, dl, lo, lse, status, BH, T,
                                            scale, causal, stream);
    }
    if (D == 64) return launch_fwd_persist<64, false>(q, nullptr, k, nullptr, v, nullptr, o, lq, lk, lv, lo, lse, status, BH, T, scale, causal, stream);
    return launch_fwd_persist<128, false>(q, nullptr, k, nullptr, v, nullptr, o, lq, lk, lv, lo, lse, status, BH, T, scale, causal, stream);
}

int bwd_core(const void* q, const void* k, const void* v, const void* o, const void* dO, const float* lse, void* dq, void* dk, void* dv,
             const ib200_layout* const lay[8], int B, int H, int T, int D, float scale, int causal, int dtype, int math_mode,
             void* workspace, size_t workspace_bytes, bool use_static, cudaStream_t stream) {
    if (!q || !k || !v || !o || !dO || !lse || !dq || !dk || !dv) return IB200_ERR_INVALID_ARGUMENT;
    int rc = check_common(B, H, T, D, dtype, math_mode, causal);
    if (rc != IB200_OK) return rc;
    if (!(scale > 0.f) || !isfinite(scale)) return IB200_ERR_INVALID_ARGUMENT;
    if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o) || !aligned16(dO) || !aligned16(lse) ||
        !aligned16(dq) || !aligned16(dk) || !aligned16(dv))
        return IB200_ERR_MISALIGNED;
    const long BH = static_cast<long>(B) * H;
    const long N = BH * T * D;
    const bool f32 = dtype == IB200_DTYPE_F32;
    BwdLayouts L;
    RowLayout* dst[8] = {&L.q, &L.k, &L.v, &L.o, &L.dO, &L.dq, &L.dk, &L.dv};
    for (int i = 0; i < 8; ++i)
        if ((rc = resolve_layout(lay[i], H, T, D, f32, dst[i]))) return rc;
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    if (use_static) {
        if (bwd_ws_bytes(N, BH, T, f32) > static_cast<size_t>(IB200_STATIC_SCRATCH_BYTES)) return IB200_ERR_TOO_LARGE;
    } else if (!workspace || !aligned16(workspace) || workspace_bytes < bwd_ws_bytes(N, BH, T, f32)) {
        return IB200_ERR_WORKSPACE;
    }
    rc = device_ok();
    if (rc != IB200_OK) return rc;
    if (use_static) {
        void* scratch = nullptr;
        rc = static_scratch(&scratch);
        if (rc != IB200_OK) return rc;
        ws = static_cast<uint8_t*>(scratch);
    }
    // launch_bwd_all clears the header and the dQ accumulator on `stream` and rewrites every other part of the
    // scratch it reads, so stale contents of an earlier call (static scratch is shared) are never consumed
    return launch_bwd_all(q, k, v, o, dO, lse, dq, dk, dv, L, BH, T, D, scale, causal, f32, ws, stream);
}

}  // namespace

extern "C" {

int ib200_version(void) { return 1001; }

int ib200_attn_item_order(int pass, int B, int H, int T, int D, int sm_count, int* heads, int* units, int capacity, int* n_groups) {
    if (B <= 0 || H <= 0 || T <= 0 || sm_count <= 0 || capacity < 0 || (capacity > 0 && (!heads || !units))) return -IB200_ERR_INVALID_ARGUMENT;
    if (D != 64 && D != 128) return -IB200_ERR_UNSUPPORTED;
    if (pass != IB200_PASS_FWD && pass != IB200_PASS_BWD) return -IB200_ERR_INVALID_ARGUMENT;
    const long BH = static_cast<long>(B) * H;
    const bool fwd = pass == IB200_PASS_FWD;
    const int per_head = fwd ? (T + 255) / 256 : (T + 127) / 128;       // query-tile pairs / key tiles
    const long items = per_head * BH;
    if (BH > 65535 || items > 0x7fffffffL) return -IB200_ERR_UNSUPPORTED;
    const int groups = persist_head_groups(sm_count, per_head, BH, static_cast<size_t>(T) * D * (fwd ? 4 : 8));
    if (n_groups) *n_groups = groups;
    const HeadGroups hg{static_cast<int>(BH), groups, per_head};
    for (long i = 0; i < items && i < capacity; ++i) {
        int rank, bh;
        locate_item(hg, static_cast<int>(i), rank, bh);
        heads[i] = bh;
        units[i] = fwd ? per_head - 1 - rank : rank;                      // the longest walk first: last pair / first key tile
    }
    return static_cast<int>(items);
}

int ib200_last_cuda_error(void) { return g_last_cuda_error; }

int ib200_attn_set_timing_events(ib200_event_t fwd_start, ib200_event_t fwd_stop, ib200_event_t bwd_start, ib200_event_t bwd_stop) {
    g_ev[0] = reinterpret_cast<cudaEvent_t>(fwd_start);
    g_ev[1] = reinterpret_cast<cudaEvent_t>(fwd_stop);
    g_ev[2] = reinterpret_cast<cudaEvent_t>(bwd_start);
    g_ev[3] = reinterpret_cast<cudaEvent_t>(bwd_stop);
    return IB200_OK;
}

static int cast_common(const void* src, void* dst, size_t n) {
    if (!src || !dst || n == 0) return IB200_ERR_INVALID_ARGUMENT;
    if (n % 8) return IB200_ERR_UNSUPPORTED;
    if (!aligned16(src) || !aligned16(dst)) return IB200_ERR_MISALIGNED;
    return device_ok();
}

int ib200_cast_f32_to_bf16(const float* src, void* dst, size_t n, ib200_stream_t stream) {
    const int rc = cast_common(src, dst, n);
    if (rc != IB200_OK) return rc;
    const long n8 = static_cast<long>(n / 8);
    long blocks = n8 / kAuxThreads + 1;
    if (blocks > kAuxBlocks) blocks = kAuxBlocks;
    cast_f32_bf16_kernel<<<static_cast<int>(blocks), kAuxThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const float4*>(src), static_cast<uint4*>(dst), n8);
    return cuda_ok(cudaGetLastError()) ? IB200_OK : IB200_ERR_CUDA;
}

int ib200_cast_bf16_to_f32(const void* src, float* dst, size_t n, ib200_stream_t stream) {
    const int rc = cast_common(src, dst, n);
    if (rc != IB200_OK) return rc;
    const long n8 = static_cast<long>(n / 8);
    long blocks = n8 / kAuxThreads + 1;
    if (blocks > kAuxBlocks) blocks = kAuxBlocks;
    cast_bf16_f32_kernel<<<static_cast<int>(blocks), kAuxThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(src), reinterpret_cast<float4*>(dst), n8);
    return cuda_ok(cudaGetLastError()) ? IB200_OK : IB200_ERR_CUDA;
}

const char* ib200_status_string(int status) {
    switch (status) {
        case IB200_OK: return "ok";
        case IB200_ERR_INVALID_ARGUMENT: return "invalid argument";
        case IB200_ERR_UNSUPPORTED: return "unsupported shape, dtype or mode";
        case IB200_ERR_MISALIGNED: return "pointer not 16-byte aligned";
        case IB200_ERR_WORKSPACE: return "workspace missing or too small";
        case IB200_ERR_CUDA: return "CUDA call failed";
        case IB200_ERR_DEVICE_TIMEOUT: return "device-side wait timed out";
        case IB200_ERR_NO_DEVICE: return "no sm_100 device is current";
        case IB200_ERR_TOO_LARGE: return "problem exceeds the capacity of the built-in static scratch buffer";
        default: return "unknown status";
    }
}

int ib200_attn_workspace_bytes(int B, int H, int T, int D, int dtype, int pass, size_t* out_bytes) {
    if (!out_bytes) return IB200_ERR_INVALID_ARGUMENT;
    if (pass != IB200_PASS_FWD && pass != IB200_PASS_BWD) return IB200_ERR_INVALID_ARGUMENT;
    int rc = check_common(B, H, T, D, dtype, IB200_MATH_SPLIT_BF16, 1);
    if (rc != IB200_OK) return rc;
    const long BH = static_cast<long>(B) * H;
    const long N = BH * T * D;
    const bool f32 = dtype == IB200_DTYPE_F32;
    *out_bytes = pass == IB200_PASS_FWD ? fwd_ws_bytes(N, f32) : bwd_ws_bytes(N, BH, T, f32);
    return IB200_OK;
}

int ib200_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int H, int T, int D,
                   float scale, int causal, int dtype, int math_mode, void* workspace, size_t workspace_bytes,
                   ib200_stream_t stream) {
    return fwd_core(q, k, v, o, lse, nullptr, nullptr, nullptr, nullptr, B, H, T, D, scale, causal, dtype, math_mode, workspace,
                    workspace_bytes, reinterpret_cast<cudaStream_t>(stream));
}

int ib200_attn_fwd_strided(const void* q, const void* k, const void* v, void* o, float* lse, const ib200_layout* lq,
                           const ib200_layout* lk, const ib200_layout* lv, const ib200_layout* lo, int B, int H, int T, int D,
                           float scale, int causal, int dtype, int math_mode, void* workspace, size_t workspace_bytes,
                           ib200_stream_t stream) {
    return fwd_core(q, k, v, o, lse, lq, lk, lv, lo, B, H, T, D, scale, causal, dtype, math_mode, workspace, workspace_bytes,
                    reinterpret_cast<cudaStream_t>(stream));
}

int ib200_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* dO, const float* lse,
                   void* dq, void* dk, void* dv, int B, int H, int T, int D, float scale, int causal, int dtype,
                   int math_mode, void* workspace, size_t workspace_bytes, ib200_stream_t stream) {
    const ib200_layout* lay[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    return bwd_core(q, k, v, o, dO, lse, dq, dk, dv, lay, B, H, T, D, scale, causal, dtype, math_mode, workspace, workspace_bytes,
                    false, reinterpret_cast<cudaStream_t>(stream));
}

int ib200_attn_bwd_strided(const void* q, const void* k, const void* v, const void* o, const void* dO, const float* lse,
                           void* dq, void* dk, void* dv, const ib200_layout* lq, const ib200_layout* lk, const ib200_layout* lv,
                           const ib200_layout* lo, const ib200_layout* ldo, const ib200_layout* ldq, const ib200_layout* ldk,
                           const ib200_layout* ldv, int B, int H, int T, int D, float scale, int causal, int dtype, int math_mode,
                           void* workspace, size_t workspace_bytes, ib200_stream_t stream) {
    const ib200_layout* lay[8] = {lq, lk, lv, lo, ldo, ldq, ldk, ldv};
    return bwd_core(q, k, v, o, dO, lse, dq, dk, dv, lay, B, H, T, D, scale, causal, dtype, math_mode, workspace, workspace_bytes,
                    false, reinterpret_cast<cudaStream_t>(stream));
}

int ib200_attn_bwd_static(const void* q, const void* k, const void* v, const void* o, const void* dO, const float* lse,
                          void* dq, void* dk, void* dv, int B, int H, int T, int D, float scale, int causal, int dtype,
                          int math_mode, ib200_stream_t stream) {
    const ib200_layout* lay[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    return bwd_core(q, k, v, o, dO, lse, dq, dk, dv, lay, B, H, T, D, scale, causal, dtype, math_mode, nullptr, 0, true,
                    reinterpret_cast<cudaStream_t>(stream));
}

int ib200_gemm_bf16(const void* a, const void* b, void* c, const float* bias, int M, int N, int K, int a_transposed,
                    int b_transposed, ib200_stream_t stream) {
    return gemm_dispatch(a, b, c, bias, M, N, K, a_transposed, b_transposed, reinterpret_cast<cudaStream_t>(stream));
}

int ib200_linear_fwd(const void* x, const void* w, const float* bias, void* y, int M, int K, int N, ib200_stream_t stream) {
    return gemm_dispatch(x, w, y, bias, M, N, K, 0, 0, reinterpret_cast<cudaStream_t>(stream));
}

int ib200_linear_bwd(const void* x, const void* w, const void* dy, void* dx, void* dw, float* db, int M, int K, int N,
                     ib200_stream_t stream_) {
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    if (!x || !w || !dy) return IB200_ERR_INVALID_ARGUMENT;
    int rc = IB200_OK;
    // dx[M,K] = dy[M,N] w^T: w is stored [K, N], i.e. the "B" of this product stored [N_out = K rows, contraction N contiguous]
    if (dx && (rc = gemm_dispatch(dy, w, dx, nullptr, M, K, N, 0, 1, stream))) return rc;
    // dw[K,N] = x^T dy: x is stored [M, K], i.e. the "A" of this product stored [contraction M rows, K contiguous]
    if (dw && (rc = gemm_dispatch(x, dy, dw, nullptr, K, N, M, 1, 0, stream))) return rc;
    if (db) {
        if (N % 8) return IB200_ERR_UNSUPPORTED;
        // row slabs so that the grid covers the SMs a few times over; the slabs meet in fp32 atomics on a zeroed db
        int slabs = (4 * 148 + (N + 63) / 64 - 1) / ((N + 63) / 64);
        if (slabs > (M + 255) / 256) slabs = (M + 255) / 256;
        if (slabs < 1) slabs = 1;
        const int rows_per_block = ((M + slabs - 1) / slabs + 7) / 8 * 8;
        if (!cuda_ok(cudaMemsetAsync(db, 0, static_cast<size_t>(N) * 4, stream))) return IB200_ERR_CUDA;
        colsum_bf16_kernel<<<dim3((N + 63) / 64, (M + rows_per_block - 1) / rows_per_block), 256, 0, stream>>>(
            static_cast<const __nv_bfloat16*>(dy), db, M, N, rows_per_block);
        if (!cuda_ok(cudaGetLastError())) return IB200_ERR_CUDA;
    }
    return IB200_OK;
}

static int read_and_clear_status(void* header, cudaStream_t stream, int* device_code) {
    int hdr[4] = {0, 0, 0, 0};
    if (!cuda_ok(cudaMemcpyAsync(hdr, header, sizeof(hdr), cudaMemcpyDeviceToHost, stream))) return IB200_ERR_CUDA;
    if (!cuda_ok(cudaStreamSynchronize(stream))) return IB200_ERR_CUDA;
    // a caller workspace that no call has prepared yet holds no status
    const int code = (hdr[3] == kHeaderMagic || header_is_builtin(header)) ? hdr[0] : 0;
    if (device_code) *device_code = code;
    if (code == 0) return IB200_OK;
    if (!cuda_ok(cudaMemsetAsync(header, 0, sizeof(int), stream))) return IB200_ERR_CUDA;      // reported once
    return IB200_ERR_DEVICE_TIMEOUT;
}

int ib200_attn_check(const void* workspace, ib200_stream_t stream, int* device_code) {
    if (!workspace) return IB200_ERR_INVALID_ARGUMENT;
    return read_and_clear_status(const_cast<void*>(workspace), reinterpret_cast<cudaStream_t>(stream), device_code);
}

int ib200_selftest_wait_expiry(void* workspace, size_t workspace_bytes, unsigned limit_us, ib200_stream_t stream_) {
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    if (!workspace || !aligned16(workspace) || workspace_bytes < kHeaderBytes) return IB200_ERR_WORKSPACE;
    if (limit_us == 0 || limit_us > 100000u) return IB200_ERR_INVALID_ARGUMENT;
    int rc = device_ok();
    if (rc != IB200_OK) return rc;
    if ((rc = prepare_header(workspace, stream))) return rc;
    IB200_SET_BOUNDS(0, 0, 0, 0, 0, 1, 32, static_cast<int*>(workspace), stream);
    wait_expiry_probe_kernel<<<1, 128, 0, stream>>>(static_cast<int*>(workspace), 1000ull * limit_us);
    return launch_status();
}

int ib200_attn_check_static(ib200_stream_t stream, int* device_code) {
    int rc = device_ok();
    if (rc != IB200_OK) return rc;
    void* builtin = nullptr;
    if ((rc = static_scratch(&builtin)) != IB200_OK) return rc;
    return read_and_clear_status(builtin, reinterpret_cast<cudaStream_t>(stream), device_code);
}

}  // extern "C"
