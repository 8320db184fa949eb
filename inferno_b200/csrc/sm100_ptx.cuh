// Thin inline-PTX layer for Blackwell (sm_100a): mbarriers, TMA tile copies,
// tensor memory (TMEM) management, tcgen05 MMA issue/commit and TMEM<->register
// moves, plus the shared-memory and instruction descriptors the MMAs consume.
// Everything here is device-side except the tensor-map encoder at the bottom.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ib200 {

// ----------------------------------------------------------------------------
// Bounded waits.  No wait in this library spins forever: after kSpinLimit failed
// polls, or kWaitLimitNs of wall-clock time (a failed try_wait may itself suspend the
// thread for a system-dependent while, so a poll count alone does not bound time),
// the waiter raises the CTA-wide abort flag and records a code in the kernel's global
// status word; every later wait in that CTA returns at once, the CTA runs to its
// normal tear-down (TMEM freed) and the host reports an error.
// ----------------------------------------------------------------------------
constexpr uint32_t kSpinLimit = 1u << 24;
#ifdef IB200_BOUNDS
constexpr unsigned long long kWaitLimitNs = 50000000ull;        // checked build: a skipped copy leaves its barrier waiting; give up after 50 ms
#else
constexpr unsigned long long kWaitLimitNs = 4000000000ull;      // 4 s: three orders of magnitude above the longest kernel
#endif

__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

enum : int {
    kDevOk = 0,
    kDevTimeoutBase = 100,   // 100 + site id of the wait that gave up
    kDevBoundsBase = 200,    // 200 + kind of access that failed its range check (checked build only)
};

// ----------------------------------------------------------------------------
// Checked build (-DIB200_BOUNDS): every TMA copy, tensor-memory access and swizzled shared-memory
// store below first checks its coordinates / addresses against the extents the host put into
// c_bounds before the launch.  A violation records kDevBoundsBase + kind in the status word and
// the access is SKIPPED -- nothing traps or asserts; a skipped load leaves its barrier waiting,
// the bounded wait gives up, and the kernel runs to its normal tear-down.  The regular build
// compiles none of this.
// ----------------------------------------------------------------------------
#ifdef IB200_BOUNDS
struct BoundsInfo {
    int dim[4];            // extents of the operand tensors: {D, T, H, B} (attention) -- unused when relaxed
    int rows3;             // extent of the last axis of the 3-D dQ accumulator map (B*H)
    int relaxed;           // 1: only signs and alignment are checked (GEMM: every operand has its own extents)
    unsigned tmem_cols;    // columns this CTA allocated
    int* status;
};
__constant__ BoundsInfo c_bounds;
enum : int { kBndTmaLoad = 1, kBndTmaStore = 2, kBndTmaReduce = 3, kBndBulkLoad = 4, kBndTmemLd = 5, kBndTmemSt = 6, kBndMmaDesc = 7, kBndSwizzle = 8 };
__device__ __forceinline__ bool bounds_ok(bool cond, int kind) {
    if (cond) return true;
    if (c_bounds.status) atomicCAS(c_bounds.status, 0, kDevBoundsBase + kind);
    return false;
}
__device__ __forceinline__ bool smem_addr_ok(uint32_t saddr, uint32_t align) {
    uint32_t total;
    asm volatile("mov.u32 %0, %%total_smem_size;" : "=r"(total));
    return saddr < total && (saddr & (align - 1)) == 0;
}
__device__ __forceinline__ bool coords4_ok(int c0, int c1, int c2, int c3) {
    if (c0 < 0 || c1 < 0 || c2 < 0 || c3 < 0 || (c0 & 7)) return false;
    return c_bounds.relaxed || (c0 < c_bounds.dim[0] && c1 < c_bounds.dim[1] && c2 < c_bounds.dim[2] && c3 < c_bounds.dim[3]);
}
__device__ __forceinline__ bool tmem_addr_ok(uint32_t taddr, uint32_t ncols) {
    return (taddr & 0xffffu) + ncols <= c_bounds.tmem_cols && (taddr >> 16) < 128u;
}
#define IB200_CHECKED(cond, kind) if (!bounds_ok((cond), (kind))) return
#else
#define IB200_CHECKED(cond, kind)
#endif

struct AbortCtx {
    volatile int* cta_flag;   // shared memory, one per CTA
    int* status;              // global memory, one per launch (may be null)
};


// ---- mbarrier ---------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Non-blocking probe.  A thread that is feeding the tensor pipe loses about 70 cycles of issue to a try_wait even
// when the phase has already completed (try_wait may suspend the thread), and about 4 to a test_wait, so every
// wait probes with test_wait first and falls back to try_wait only when it really has to wait.
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Returns false if the wait was abandoned (abort already raised, or limit hit).
// The CTA abort flag lives in shared memory; it is polled only every 64th failed try so that
// spinning warps do not load the shared-memory pipe the MMAs and compute warps depend on.
// `limit_ns` is a compile-time constant at every call site of the product kernels (mbar_wait below);
// only the wait-expiry self-test kernel passes a run-time value.
__device__ __forceinline__ bool mbar_wait_limit(uint64_t* bar, uint32_t parity, const AbortCtx& ab, int site, unsigned long long limit_ns) {
    if (mbar_test_wait(bar, parity)) return true;
    uint32_t spins = 0;
    unsigned long long t_start = 0;
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((++spins & 63u) == 0) {
            if (*ab.cta_flag != 0) return false;
            const unsigned long long now = global_timer_ns();
            if (t_start == 0) t_start = now;
            if (spins > kSpinLimit || now - t_start > limit_ns) {
                *ab.cta_flag = 1;
                if (ab.status) atomicCAS(ab.status, 0, kDevTimeoutBase + site);
                return false;
            }
        }
    }
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const AbortCtx& ab, int site) {
    return mbar_wait_limit(bar, parity, ab, site, kWaitLimitNs);
}

// ---- work items of a persistent CTA ---------------------------------------------
// Every CTA starts on item blockIdx.x and then draws items from a counter in global memory (zero at launch), so a CTA
// that drew light items simply draws more of them.  One thread of the CTA (the TMA producer, which runs furthest ahead)
// draws; the other roles read what it drew through a two-slot ring in shared memory: slot n & 1 holds the item that
// follows the CTA's n-th item, full[] (count 1) says it has been written, empty[] (count = reading warps) that every
// role has read it.  An index >= the item count ends every role's loop.
struct ItemRing {
    uint64_t* full;        // [2]
    uint64_t* empty;       // [2]
    volatile int* slot;    // [2]
};
__device__ __forceinline__ void item_ring_init(const ItemRing& r, uint32_t readers) {
    for (int s = 0; s < 2; ++s) { mbar_init(&r.full[s], 1); mbar_init(&r.empty[s], readers); }
}
// producer thread: the item after this CTA's n-th item is `next`
__device__ __forceinline__ void item_ring_publish(const ItemRing& r, int n, int next, const AbortCtx& ab) {
    const int s = n & 1;
    mbar_wait(&r.empty[s], ((n >> 1) & 1) ^ 1, ab, 14);
    r.slot[s] = next;
    mbar_arrive(&r.full[s]);
}
// reading role, called by all its (converged) lanes: the item after this CTA's n-th item
__device__ __forceinline__ int item_ring_next(const ItemRing& r, int n, const AbortCtx& ab, bool arriving_lane) {
    const int s = n & 1;
    mbar_wait(&r.full[s], (n >> 1) & 1, ab, 15);
    const int v = r.slot[s];
    __syncwarp();
    if (arriving_lane) mbar_arrive(&r.empty[s]);
    return v;
}

// The item list of a persistent attention kernel runs group by group over consecutive heads (so that the CTAs, which are
// all within about a round of each other in the list, share the tiles of few heads in L2); inside a group the unit (query
// tile pair, key tile) with the most work comes first for every head of the group, then the next unit, and so on.
// BH heads are cut into n_groups groups whose sizes differ by at most one head (the larger groups first).
struct HeadGroups {
    int BH, n_groups, units_per_head;
};
// item index -> rank of the unit inside its head (0 = first in the list) and head
__host__ __device__ __forceinline__ void locate_item(const HeadGroups& hg, int idx, int& unit_rank, int& bh) {
    const int base = hg.BH / hg.n_groups, rem = hg.BH - base * hg.n_groups;
    const int big = (base + 1) * hg.units_per_head, cut = rem * big;
    int h0, hn, r;
    if (idx < cut) {
        const int grp = idx / big;
        h0 = grp * (base + 1); hn = base + 1; r = idx - grp * big;
    } else {
        const int j = idx - cut, small = base * hg.units_per_head, grp = j / small;
        h0 = rem * (base + 1) + grp * base; hn = base; r = j - grp * small;
    }
    unit_rank = r / hn;
    bh = h0 + (r - unit_rank * hn);
}

// ---- proxy / tcgen05 fences ---------------------------------------------------
// Generic-proxy writes to shared memory -> visible to the async proxy (TMA, MMA).
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---- TMA (tiled, no multicast) ----------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// 3-D tile load global -> shared, completion on an mbarrier (transaction bytes).
// c0 is the innermost coordinate: c0 * elem_size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1, int c2) {
    IB200_CHECKED(coords4_ok(c0, c1, c2, 0) && smem_addr_ok(smem_u32(smem_dst), 1024), kBndTmaLoad);
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
// Untiled bulk copy global -> shared with mbarrier completion; both addresses 16-byte aligned,
// size a multiple of 16 bytes.
__device__ __forceinline__ void bulk_load_1d(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
    IB200_CHECKED(smem_addr_ok(smem_u32(smem_dst), 16) && (reinterpret_cast<uint64_t>(gmem_src) & 15u) == 0 && (bytes & 15u) == 0 && bytes > 0, kBndBulkLoad);
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(gmem_src)), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}
// 4-D variants: coordinates (column, token row, head, batch) over a tensor map whose head and batch
// strides are free, which is how operands that live inside a packed [B, T, 3, H, D] projection buffer
// (or any other layout with contiguous head-dim rows) are read and written in place.
__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1, int c2, int c3) {
    IB200_CHECKED(coords4_ok(c0, c1, c2, c3) && smem_addr_ok(smem_u32(smem_dst), 1024), kBndTmaLoad);
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* m, const void* smem_src, int c0, int c1, int c2, int c3) {
    IB200_CHECKED(coords4_ok(c0, c1, c2, c3) && smem_addr_ok(smem_u32(smem_src), 1024), kBndTmaStore);
    asm volatile(
        "cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
        ::"l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
// 3-D tile store shared -> global (rows outside the tensor are clipped).
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* m, const void* smem_src, int c0, int c1, int c2) {
    IB200_CHECKED(coords4_ok(c0, c1, c2, 0) && smem_addr_ok(smem_u32(smem_src), 1024), kBndTmaStore);
    asm volatile(
        "cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4}], [%1];"
        ::"l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
// 3-D tile reduction shared -> global: global[tile] += shared[tile], element type from the tensor map.
__device__ __forceinline__ void tma_reduce_add_3d(const CUtensorMap* m, const void* smem_src, int c0, int c1, int c2) {
    IB200_CHECKED(c0 == 0 && c1 >= 0 && c2 >= 0 && (c_bounds.relaxed || (c1 < c_bounds.dim[1] && c2 < c_bounds.rows3)) &&
                  smem_addr_ok(smem_u32(smem_src), 128), kBndTmaReduce);
    asm volatile(
        "cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4}], [%1];"
        ::"l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }

// ---- TMEM ----------------------------------------------------------------------
// One full warp allocates; the base address (lane 0, first column) lands in smem.
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// ---- MMA issue -----------------------------------------------------------------
// D[tmem] (+)= A[smem desc] * B[smem desc]; one thread issues for the CTA.
__device__ __forceinline__ void umma_ss_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    // operand start addresses (descriptor bits 0-13 hold address >> 4) inside the CTA's shared memory; N accumulator columns inside the allocation
    IB200_CHECKED(smem_addr_ok(static_cast<uint32_t>(adesc & 0x3fffu) << 4, 16) && smem_addr_ok(static_cast<uint32_t>(bdesc & 0x3fffu) << 4, 16) &&
                  tmem_addr_ok(d_tmem, ((idesc >> 17) & 0x3fu) << 3), kBndMmaDesc);
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem desc].
__device__ __forceinline__ void umma_ts_f16(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    IB200_CHECKED(smem_addr_ok(static_cast<uint32_t>(bdesc & 0x3fffu) << 4, 16) && tmem_addr_ok(d_tmem, ((idesc >> 17) & 0x3fu) << 3) &&
                  tmem_addr_ok(a_tmem, 8), kBndMmaDesc);
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// All MMAs issued so far by this thread arrive (once) on the mbarrier when complete.
// Implies tcgen05.fence::before_thread_sync.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// One lane of a converged warp (elect.sync).  An MMA-issuing warp that stays converged and predicates only the
// tcgen05.mma / tcgen05.commit instructions on this flag issues an MMA every ~39 cycles and commits almost for free;
// the same loop run by a single lane inside a divergent branch pays ~44 cycles per MMA and ~44 more per commit.
__device__ __forceinline__ bool elect_one_lane() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
}

// ---- descriptors ---------------------------------------------------------------
constexpr uint32_t kMajorK = 0, kMajorMN = 1;
constexpr uint32_t kFmtBF16 = 1;

// Instruction descriptor for kind::f16 with fp32 accumulation.
__host__ __device__ constexpr uint32_t make_idesc(uint32_t fmt, uint32_t M, uint32_t N, uint32_t a_major, uint32_t b_major) {
    return (1u << 4)                 // accumulator format: f32
           | (fmt << 7)              // A format
           | (fmt << 10)             // B format
           | (a_major << 15) | (b_major << 16)
           | ((N >> 3) << 17) | ((M >> 4) << 24);
}

// Shared-memory matrix descriptor, 128-byte swizzle (matches TMA SWIZZLE_128B;
// swizzle atoms are 8 rows x 128 bytes and must start on 1024-byte boundaries).
//   K-major  (rows = M or N index, 128 contiguous bytes of K per row):
//       sbo = byte distance between 8-row groups; lbo unused.
//   MN-major (rows = K index, 128 contiguous bytes of M or N per row):
//       lbo = byte distance between 128-byte column panels along M/N,
//       sbo = byte distance between 8-row groups along K.
// The descriptor is built from two words, so that an MMA issue loop pays one 32-bit add per operand:
// the high word is a constant for every 128B-swizzled operand with 1024-byte 8-row groups, and the
// low word is (address >> 4) | (lbo >> 4) << 16, to which a byte offset adds as (offset >> 4).
constexpr uint32_t kSdescHiSw128 = (1024u >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint32_t sdesc_lo(uint32_t saddr, uint32_t lbo_bytes) {
    return ((saddr & 0x3FFFFu) >> 4) | ((lbo_bytes >> 4) << 16);
}
__device__ __forceinline__ uint64_t sdesc_join(uint32_t lo) {
    uint64_t d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(kSdescHiSw128));
    return d;
}

// Byte offset of 16-byte chunk `chunk16` of row `row` inside a 128B-swizzled panel
// whose rows are 128 bytes (the layout TMA SWIZZLE_128B produces).
__host__ __device__ __forceinline__ uint32_t sw128_offset(uint32_t row, uint32_t chunk16) {
    return row * 128u + ((chunk16 ^ (row & 7u)) << 4);
}

// 16-byte store into a 128B-swizzled panel ([rows x 128 bytes], 1024-byte aligned).
__device__ __forceinline__ void st_shared_sw128(uint8_t* panel, uint32_t row, uint32_t chunk16, uint4 v) {
    IB200_CHECKED(row < 256u && chunk16 < 8u && smem_addr_ok(smem_u32(panel), 1024), kBndSwizzle);
    *reinterpret_cast<uint4*>(panel + sw128_offset(row, chunk16)) = v;
}

// ---- TMEM <-> registers --------------------------------------------------------
// 32x32b shape: the warp reads 32 lanes (its quarter: lanes 32*(warp%4)..+31),
// thread i gets lane i, N consecutive 32-bit columns.
__device__ __forceinline__ void tmem_ld_x32(uint32_t taddr, uint32_t (&r)[32]) {
#ifdef IB200_BOUNDS
    if (!bounds_ok(tmem_addr_ok(taddr, 32), kBndTmemLd)) {
#pragma unroll
        for (int e = 0; e < 32; ++e) r[e] = 0u;
        return;
    }
#endif
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st_x32(uint32_t taddr, const uint32_t (&r)[32]) {
    IB200_CHECKED(tmem_addr_ok(taddr, 32), kBndTmemSt);
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31};"
        ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]),
          "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st_x16(uint32_t taddr, const uint32_t (&r)[16]) {
    IB200_CHECKED(tmem_addr_ok(taddr, 16), kBndTmemSt);
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%16], "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15};"
        ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ---- small numeric helpers -----------------------------------------------------
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
// Packed fp32x2 arithmetic (one instruction for two lanes of fp32 math).
// three-input maximum (one instruction on sm_100)
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack_f32x2(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t ffma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t fadd2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t fmul2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
}  // namespace ib200
