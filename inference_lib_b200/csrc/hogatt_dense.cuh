// Dense fragment attention on the 5th-generation tensor cores (tcgen05): the path for calls with many query
// rows per kv head -- W workers x G grouped heads x S-token chunks >= 128 rows -- where the op is bound by the
// tensor pipe instead of HBM (16-token causal chunks of 8 workers with GQA 8 are 1,024 rows per kv head: about
// 1,000 flop per K/V byte).
//
// Same decomposition, workspace format and merge step as the other attention kernels (hogatt_plan.h): a unit is
// (block of 128 query rows, kv head), its visible keys are tiles of 128 keys that never straddle a fragment, a
// persistent grid of one CTA per SM walks balanced contiguous tile ranges and leaves unnormalised partial
// results, merge_kernel folds them.  What differs is how a tile is computed:
//
//   * Queries arrive ALREADY ROTATED as [F, W, Hq, S, E] (the rotated-query output of the fused op, written by
//     rope_kernel just before; or the caller's own for the pre-rotated entry point).  A 128-row query tile of one
//     fragment and kv head is one 5-D TMA box of that tensor.
//   * K, V and Q tiles are fetched by TMA (cp.async.bulk.tensor, one tensor map per fragment, encoded on the
//     host) into shared memory in the 128-byte-swizzled layout the tensor core reads directly.
//   * S = Q K^T (128 x 128 x 128) and O += P V (128 x 128 x 128) are tcgen05.mma instructions issued by one
//     thread; S (two buffers), P and O live in tensor memory.  The softmax warps pull S out of tensor memory
//     (tcgen05.ld), mask, exponentiate, write P as bf16/f16 back into tensor memory (tcgen05.st) -- the second MMA
//     takes its A operand from there: no trip of P through shared memory, no proxy fence, and room for deeper K / V
//     rings (measured 166 -> 157 us per 1,024-row group) -- and keep the running max and sum in registers.  (Measured
//     and not kept: the query tile as a tensor-memory operand too, 176 us; two query buffers with a segment-ahead fetch
//     at the price of a two-stage K ring, +4 us; two softmax groups taking the tiles in turn, one thread per row,
//     +20 us; programmatic dependent launch behind the rotation kernel, +3 us; half of a tile's exponentials as a cubic on
//     the FMA pipe instead of the special-function unit, +7 us: the softmax threads are bound by issue slots and
//     latency, not by ex2 throughput.)  O is rescaled in tensor memory only when a row's
//     max has grown by more than 2^8 since the scale it is stored at (then exp2 arguments stay below 8 and
//     nothing overflows); the stored scale travels with the partial result, so the merge is exact.
//
// Warp roles (352 threads): warps 0-7 softmax, warp 8 issues the K/V copies, warp 9 allocates tensor memory, issues
// the Q copies and the S MMAs, warp 10 issues the PV MMAs.  Softmax warps w and w + 4 share the 32 query rows of tensor-memory lanes
// 32 (w % 4) ... + 31 and split the 128 columns of S (keys) and of O between them: two warps per scheduler hide each
// other's latencies, and a thread keeps 64 scores in registers.  Both derive the same row maximum -- each also
// reads the other half's scores for that, which costs two more tensor-memory loads and no synchronisation -- so
// the probabilities of a row share one scale.  Every wait is bounded.
//
// The reference has no counterpart: its kernel gives every (kv head, worker, token) its own CTAs and re-reads the
// KV once per (worker, token) on CUDA cores (src/kernels/kernel_v21.cuh:62-66,957-964).
#pragma once
#include <cuda.h>

#include "hogatt_device.cuh"

namespace hogatt {

constexpr int kDenseMaxFragments = 16;      // tensor maps travel in the kernel arguments
constexpr int kDenseRows = 128;             // query rows per CTA (MMA M)
constexpr int kDenseTile = 128;             // keys per tile (MMA N of S, K of PV)
// Softmax warps per 32-row group: each takes 128 / SPLIT columns of every row.  (Measured on the 1,024-row shape: two
// beat four -- every warp re-reads the whole row for the maximum, so four warps issue 1.7 times the instructions.)
constexpr int kDenseSplit = 2;
constexpr int kDenseSoftmaxWarps = 4 * kDenseSplit;
constexpr int kDenseThreads = (kDenseSoftmaxWarps + 3) * 32;

struct alignas(64) DenseMaps {
    CUtensorMap q;                          // [F, W, Hkv, G*S, E] view of the rotated queries
    CUtensorMap k[kDenseMaxFragments];      // [Hkv, rows, E] per fragment
    CUtensorMap v[kDenseMaxFragments];      // [Hkv, rows, Ev]
};

struct DenseCfg {
    static constexpr int HD = 128;
    static constexpr int ATOM_BYTES = 128 * 128;            // [128 rows][64 16-bit columns], rows of 128 bytes, swizzled
    static constexpr int TILE_BYTES = 2 * ATOM_BYTES;       // a 128 x 128 operand tile: two column halves
    static constexpr int NK = 3, NV = 3;                    // K ring, V ring
    static constexpr int OFF_Q = 0;
    static constexpr int OFF_K = OFF_Q + TILE_BYTES;
    static constexpr int OFF_V = OFF_K + NK * TILE_BYTES;
    static constexpr int OFF_BAR = OFF_V + NV * TILE_BYTES;                 // 224 KiB of tiles
    // barriers: q_full, k_full[NK], k_empty[NK], v_full[NV], v_empty[NV], s_full[2], s_free[2], p_full, o_done, l_ready[4]
    static constexpr int NBAR = 1 + 2 * NK + 2 * NV + 2 + 2 + 1 + 1 + 4;
    static constexpr int OFF_MISC = OFF_BAR + NBAR * 8;                     // tmem base, abort flag
    static constexpr int OFF_PLAN = OFF_MISC + 16;                          // vis[F], pre[F + 1]
    static constexpr int TMEM_COLS = 512;
    static constexpr int COL_O = 0, COL_S0 = 128, COL_S1 = 256;
    static constexpr int COL_P = 384;           // 64 columns: P, two 16-bit probabilities per 32-bit column
    static constexpr int COL_L = 448;           // 2 x 4 columns: the column groups' shares of the row sums, handed over at a flush
};

__host__ __device__ inline size_t dense_smem_bytes(int F) {
    return 1024 /* alignment slack: swizzled tiles start on 1 KiB boundaries */ + DenseCfg::OFF_PLAN + ((size_t)2 * F + 1) * 4;
}

// ---- tcgen05 / TMA wrappers -------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// arrive on `bar` once every MMA this thread has issued so far has completed
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem], 128 x N x 16, fp32 accumulate
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem]: A is 128 rows (lanes) x 16 k (8 columns, two 16-bit elements each, lower k in the low half)
__device__ __forceinline__ void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Shared-memory matrix descriptor, 128-byte swizzle: start address, leading / stride byte offsets in 16-byte units,
// descriptor version 1 (bits 46-47), layout type 2 = SWIZZLE_128B (bits 61-63).
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo_bytes >> 4) << 16) | ((uint64_t)(sbo_bytes >> 4) << 32) |
           (1ull << 46) | (2ull << 61);
}
// Instruction descriptor, kind::f16: fp32 accumulator (bits 4-5 = 1), A/B format (bits 7-9, 10-12: 0 f16, 1 bf16),
// A K-major, B K-major or MN-major (bit 16), N >> 3 (bits 17-22), M >> 4 (bits 24-28).
template <class T>
__host__ __device__ constexpr uint32_t umma_idesc(bool b_mn_major, int m, int n) {
    const uint32_t fmt = sizeof(T) == 2 && std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
    return (1u << 4) | (fmt << 7) | (fmt << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, int c4,
                                            uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], [%7];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4), "r"(bar)
        : "memory");
}

// 32 consecutive fp32 columns of this thread's tensor-memory lane
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t* r = reinterpret_cast<uint32_t*>(v);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float (&v)[32]) {
    const uint32_t* r = reinterpret_cast<const uint32_t*>(v);
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
          "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
          "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
// 2^x, the hardware approximation (about two units in the last place); -inf gives 0
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ void tmem_st1(uint32_t taddr, float v) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x1.b32 [%0], {%1};" ::"r"(taddr), "r"(__float_as_uint(v)) : "memory");
}
__device__ __forceinline__ void tmem_ld4(uint32_t taddr, float (&v)[4]) {
    uint32_t* r = reinterpret_cast<uint32_t*>(v);
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ---- the walk over this CTA's tiles, identical in every role ----------------------------------------------------
struct DenseTile {
    int u, f, tok0, ntok, hkv, rb;
    bool first_of_unit;     // first tile of this CTA's share of the unit: O starts from zero
    bool last_of_unit;      // last tile of the share: the partial result is due
    bool new_segment;       // the query tile differs from the previous tile's (other fragment or other unit)
};
struct DenseWalk {
    const int *vis, *pre;
    int F, Hkv, TH, j, fscan, prev_u, prev_f;
    int64_t u, t, t1;
    __device__ __forceinline__ DenseWalk(const int* vis_, const int* pre_, int F_, int Hkv_, int64_t t0, int64_t t1_)
        : vis(vis_), pre(pre_), F(F_), Hkv(Hkv_), TH(pre_[F_]), fscan(0), prev_u(-1), prev_f(-1), t(t0), t1(t1_) {
        u = TH > 0 ? t0 / TH : 0;
        j = (int)(t0 - u * TH);
    }
    __device__ __forceinline__ bool done() const { return t >= t1; }
    __device__ __forceinline__ DenseTile next() {
        DenseTile d;
        while (j >= pre[fscan + 1]) ++fscan;
        d.u = (int)u;
        d.f = fscan;
        d.tok0 = (j - pre[fscan]) * kDenseTile;
        d.ntok = min(kDenseTile, vis[fscan] - d.tok0);
        d.hkv = d.u % Hkv;
        d.rb = d.u / Hkv;
        d.first_of_unit = d.u != prev_u;
        d.new_segment = d.u != prev_u || d.f != prev_f;
        d.last_of_unit = (j == TH - 1) || (t == t1 - 1);
        prev_u = d.u;
        prev_f = d.f;
        ++t;
        if (++j == TH) {
            j = 0;
            ++u;
            fscan = 0;
        }
        return d;
    }
};

template <class T>
__global__ void __launch_bounds__(kDenseThreads, 1)
dense_attention_kernel(const __grid_constant__ KernelArgs a, const __grid_constant__ DenseMaps maps) {
    using C = DenseCfg;
    extern __shared__ unsigned char smem_dyn[];
    unsigned char* base = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
    const uint32_t sbase = smem_u32(base);
    const uint32_t bars = sbase + C::OFF_BAR;
    const uint32_t q_full = bars, k_full = q_full + 8, k_empty = k_full + 8 * C::NK, v_full = k_empty + 8 * C::NK,
                   v_empty = v_full + 8 * C::NV, s_full = v_empty + 8 * C::NV, s_free = s_full + 16, p_full = s_free + 16,
                   o_done = p_full + 8, l_ready = o_done + 8;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base + C::OFF_MISC);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(base + C::OFF_MISC + 8);
    int* vis = reinterpret_cast<int*>(base + C::OFF_PLAN);
    int* pre = vis + a.F;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    HOGATT_TL_DECL;

    if (tid == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < C::NK; ++s) {
            mbar_init(k_full + 8 * s, 1);
            mbar_init(k_empty + 8 * s, 1);
        }
        for (int s = 0; s < C::NV; ++s) {
            mbar_init(v_full + 8 * s, 1);
            mbar_init(v_empty + 8 * s, 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(s_full + 8 * s, 1);
            mbar_init(s_free + 8 * s, kDenseSoftmaxWarps);      // one arrival per softmax warp
        }
        mbar_init(p_full, kDenseSoftmaxWarps);
        mbar_init(o_done, 1);
        for (int s = 0; s < 4; ++s) mbar_init(l_ready + 8 * s, kDenseSplit - 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_proxy_async_smem();
    }
    if (warp == kDenseSoftmaxWarps + 1) tmem_alloc(smem_u32(tmem_slot), C::TMEM_COLS);
    if (a.host_plan) {
        if (warp == 0) host_tile_prefix(a, kDenseTile, vis, pre);
        tc_fence_before();
        __syncthreads();
    } else {
        tc_fence_before();
        build_tile_prefix(a, kDenseTile, vis, pre);        // ends with __syncthreads()
    }
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    const int TH = pre[a.F];
    const int units = a.row_blocks * a.Hkv;
    const int64_t N = (int64_t)units * TH;
    const int ctas = a.host_plan ? a.plan_ctas : effective_ctas(N, gridDim.x);
    if (!a.host_plan && blockIdx.x == 0 && tid == 0) {
        a.header[0] = TH;
        a.header[1] = ctas;
    }
    int64_t t0 = 0, t1 = 0;
    if ((int)blockIdx.x < ctas) {
        t0 = cta_first_tile(blockIdx.x, N, ctas);
        t1 = cta_first_tile(blockIdx.x + 1, N, ctas);
    }
    const int GS = a.G * a.S;

    if (warp == kDenseSoftmaxWarps) {
        // ============================== K / V copies ==============================
        if (lane == 0) {
            DenseWalk walk(vis, pre, a.F, a.Hkv, t0, t1);
            bool ok = true;
            for (int it = 0; !walk.done() && ok; ++it) {
                const DenseTile d = walk.next();
                const int ks = it % C::NK, vs = it % C::NV;
                ok = mbar_wait_bounded(k_empty + 8 * ks, (((uint32_t)(it / C::NK)) & 1u) ^ 1u, abort_flag, a.status,
                                       STATUS_WAIT_EMPTY_TIMEOUT);
                if (!ok) break;
                mbar_arrive_expect_tx(k_full + 8 * ks, C::TILE_BYTES);
                const uint32_t kdst = sbase + C::OFF_K + ks * C::TILE_BYTES;
                tma_load_3d(kdst, &maps.k[d.f], 0, d.tok0, d.hkv, k_full + 8 * ks);
                tma_load_3d(kdst + C::ATOM_BYTES, &maps.k[d.f], 64, d.tok0, d.hkv, k_full + 8 * ks);
                ok = mbar_wait_bounded(v_empty + 8 * vs, (((uint32_t)(it / C::NV)) & 1u) ^ 1u, abort_flag, a.status,
                                       STATUS_WAIT_EMPTY_TIMEOUT);
                if (!ok) break;
                mbar_arrive_expect_tx(v_full + 8 * vs, C::TILE_BYTES);
                const uint32_t vdst = sbase + C::OFF_V + vs * C::TILE_BYTES;
                tma_load_3d(vdst, &maps.v[d.f], 0, d.tok0, d.hkv, v_full + 8 * vs);
                tma_load_3d(vdst + C::ATOM_BYTES, &maps.v[d.f], 64, d.tok0, d.hkv, v_full + 8 * vs);
            }
        }
    } else if (warp == kDenseSoftmaxWarps + 1) {
        // ============================== Q copies and the S MMAs ==============================
        // Issuing a tcgen05.mma costs the issuing thread some 60-70 cycles, sixteen of them per tile about as long as
        // the tensor pipe needs to execute them -- so the two GEMMs of a tile are issued by two threads that only meet at
        // barriers: this one runs ahead with S = Q K^T, the next warp follows the softmax warps with O += P V.
        if (lane == 0) {
            constexpr uint32_t IDESC_S = umma_idesc<T>(false, kDenseRows, kDenseTile);
            const uint32_t q_smem = sbase + C::OFF_Q;
            uint32_t q_phase = 0;
            // the matrix descriptors are built once (a k-step only moves the start-address field: +32 bytes inside a
            // 64-column swizzle atom, +16 KiB to the second atom)
            const uint64_t q_desc = umma_desc(q_smem, 16, 1024);
            uint64_t k_desc[C::NK];
#pragma unroll
            for (int i = 0; i < C::NK; ++i) k_desc[i] = umma_desc(sbase + C::OFF_K + i * C::TILE_BYTES, 16, 1024);
            DenseWalk walk(vis, pre, a.F, a.Hkv, t0, t1);
            bool ok = true;
            for (int it = 0; !walk.done() && ok; ++it) {
                const DenseTile d = walk.next();
                const int ks = it % C::NK, sb = it & 1;
                if (d.new_segment) {
                    // the query tile changes: S_{it-1}, the last reader of the old one, must have finished
                    if (it > 0)
                        ok = mbar_wait_bounded(s_full + 8 * ((it - 1) & 1), ((uint32_t)((it - 1) >> 1)) & 1u, abort_flag, a.status,
                                               STATUS_WAIT_SYNC_TIMEOUT);
                    if (!ok) break;
                    const int r0 = d.rb * kDenseRows;
                    mbar_arrive_expect_tx(q_full, C::TILE_BYTES);
                    tma_load_5d(q_smem, &maps.q, 0, r0 % GS, d.hkv, r0 / GS, d.f, q_full);
                    tma_load_5d(q_smem + C::ATOM_BYTES, &maps.q, 64, r0 % GS, d.hkv, r0 / GS, d.f, q_full);
                    ok = mbar_wait_bounded(q_full, q_phase, abort_flag, a.status, STATUS_WAIT_FULL_TIMEOUT);
                    q_phase ^= 1u;
                    if (!ok) break;
                }
                // S_it = Q K^T into S buffer it & 1 (K ring stage it % NK); the stage is handed back when the MMAs are done
                ok = mbar_wait_bounded(k_full + 8 * ks, ((uint32_t)(it / C::NK)) & 1u, abort_flag, a.status, STATUS_WAIT_FULL_TIMEOUT) &&
                     mbar_wait_bounded(s_free + 8 * sb, (((uint32_t)(it >> 1)) & 1u) ^ 1u, abort_flag, a.status, STATUS_WAIT_SYNC_TIMEOUT);
                if (!ok) break;
                tc_fence_after();
                const uint64_t kd = ks == 0 ? k_desc[0] : (ks == 1 ? k_desc[1] : k_desc[2]);
                const uint32_t d_tmem = tmem + (sb ? C::COL_S1 : C::COL_S0);
#pragma unroll
                for (int kk = 0; kk < C::HD / 16; ++kk) {
                    const uint64_t off = (uint64_t)(((kk >> 2) * C::ATOM_BYTES + (kk & 3) * 32) >> 4);
                    tc_mma(d_tmem, q_desc + off, kd + off, IDESC_S, kk > 0);
                }
                tc_commit(s_full + 8 * sb);
                tc_commit(k_empty + 8 * ks);
                HOGATT_TL(0, 3000 + it);
            }
        }
    } else if (warp == kDenseSoftmaxWarps + 2) {
        // ============================== the O += P V MMAs ==============================
        if (lane == 0) {
            constexpr uint32_t IDESC_O = umma_idesc<T>(true, kDenseRows, C::HD);
            uint64_t v_desc[C::NV];
#pragma unroll
            for (int i = 0; i < C::NV; ++i) v_desc[i] = umma_desc(sbase + C::OFF_V + i * C::TILE_BYTES, C::ATOM_BYTES, 1024);
            DenseWalk walk(vis, pre, a.F, a.Hkv, t0, t1);
            bool ok = true;
            for (int it = 0; !walk.done() && ok; ++it) {
                const DenseTile cur = walk.next();
                const int vs = it % C::NV;
                ok = mbar_wait_bounded(p_full, ((uint32_t)it) & 1u, abort_flag, a.status, STATUS_WAIT_SYNC_TIMEOUT) &&
                     mbar_wait_bounded(v_full + 8 * vs, ((uint32_t)(it / C::NV)) & 1u, abort_flag, a.status, STATUS_WAIT_FULL_TIMEOUT);
                if (!ok) break;
                tc_fence_after();
                const uint64_t vd = vs == 0 ? v_desc[0] : (vs == 1 ? v_desc[1] : v_desc[2]);
                const uint32_t acc0 = cur.first_of_unit ? 0u : 1u;
#pragma unroll
                for (int kk = 0; kk < kDenseTile / 16; ++kk) {
                    // A = P from tensor memory: 16 keys are 8 columns.  V is [key][Ev]: Ev (the MMA's N) is contiguous ->
                    // MN-major; 16 keys per step = two 8-key swizzle atoms (2 KiB)
                    tc_mma_ts(tmem + C::COL_O, tmem + C::COL_P + kk * 8, vd + (uint64_t)(kk * 2048 >> 4), IDESC_O, kk > 0 ? 1u : acc0);
                }
                tc_commit(o_done);
                tc_commit(v_empty + 8 * vs);
                HOGATT_TL(0, 2000 + it);
            }
        }
    } else {
        // ============================== softmax: SPLIT threads per query row, 128 / SPLIT columns each ==============================
        constexpr int SPLIT = kDenseSplit, COLS = kDenseTile / SPLIT;      // COLS is 32 or 64
        static_assert(COLS == 32 || COLS == 64, "a thread owns one or two 32-column tensor-memory loads");
        const int row = (warp & 3) * 32 + lane;                // row of the block == tensor-memory lane
        const int part = warp >> 2;                            // which COLS columns of S, P and O this thread owns
        const int col0 = part * COLS;
        const uint32_t lane_base = ((uint32_t)((warp & 3) * 32)) << 16;
        const float scale2 = a.l2scale;                        // scores are raw dot products; exp2((s - m) * scale2)
        const float grow_by = 8.f / scale2;                    // raw-score distance that equals a factor 2^8
        float m_run = -INFINITY, l_run = 0.f;                  // running max (raw), this thread's share of the running sum
        uint32_t nflush = 0;
        int lim = 0, vlen = 0;
        bool valid = false;
        RowId id = {0, 0, 0};
        DenseWalk walk(vis, pre, a.F, a.Hkv, t0, t1);
        bool ok = true;
        for (int it = 0; !walk.done() && ok; ++it) {
            const DenseTile d = walk.next();
            if (d.first_of_unit) {
                const int gr = d.rb * kDenseRows + row;
                valid = gr < a.rows_total;
                id = decode_row(valid ? gr : 0, a.G, a.S);
                m_run = -INFINITY;
                l_run = 0.f;
            }
            if (d.new_segment) {
                vlen = vis[d.f];
                if (a.host_plan && a.flen) vlen = min(vlen, a.flen[d.f]);
                lim = valid ? min(a.loc[(d.f * a.W + id.w) * a.S + id.s], vlen - 1) + 1 : vlen;
            }
            const int sb = it & 1;
            if (warp == 0) HOGATT_TL(1, 1000 + it);
            ok = mbar_wait_bounded(s_full + 8 * sb, ((uint32_t)(it >> 1)) & 1u, abort_flag, a.status, STATUS_WAIT_FULL_TIMEOUT);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            if (warp == 0) HOGATT_TL(1, 2000 + it);
            // ---- this thread's scores stay in registers; the other columns are only folded into the row maximum ----
            const uint32_t src = tmem + lane_base + (sb ? C::COL_S1 : C::COL_S0);
            const int nvis = lim - d.tok0;                      // keys of this tile the row sees: [0, nvis)
            float s[COLS];
            float mx0 = -INFINITY, mx1 = -INFINITY;
            {
                // every load is issued before the first is waited for (one tensor-memory round trip per tile)
                constexpr int NOTHER = (kDenseTile - COLS) / 32;
                float other[NOTHER][32];
#pragma unroll
                for (int c = 0; c < COLS / 32; ++c) tmem_ld32(src + col0 + c * 32, *reinterpret_cast<float(*)[32]>(&s[c * 32]));
#pragma unroll
                for (int c = 0; c < NOTHER; ++c) tmem_ld32(src + ((col0 + COLS + c * 32) & (kDenseTile - 1)), other[c]);
                tmem_wait_ld();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(s_free + 8 * sb);    // the next S MMA may overwrite this buffer
                if (nvis >= kDenseTile) {
#pragma unroll
                    for (int c = 0; c < NOTHER; ++c)
#pragma unroll
                        for (int k = 0; k < 32; k += 4) {
                            mx0 = max3(mx0, other[c][k], other[c][k + 1]);
                            mx1 = max3(mx1, other[c][k + 2], other[c][k + 3]);
                        }
#pragma unroll
                    for (int k = 0; k < COLS; k += 4) {
                        mx0 = max3(mx0, s[k], s[k + 1]);
                        mx1 = max3(mx1, s[k + 2], s[k + 3]);
                    }
                } else {
#pragma unroll
                    for (int c = 0; c < NOTHER; ++c) {
                        const int ob = (col0 + COLS + c * 32) & (kDenseTile - 1);
#pragma unroll
                        for (int k = 0; k < 32; ++k) mx0 = fmaxf(mx0, ob + k < nvis ? other[c][k] : -INFINITY);
                    }
#pragma unroll
                    for (int k = 0; k < COLS; ++k) {
                        s[k] = col0 + k < nvis ? s[k] : -INFINITY;
                        mx1 = fmaxf(mx1, s[k]);
                    }
                }
            }
            if (warp == 0) HOGATT_TL(1, 3000 + it);
            const float mx = fmaxf(mx0, mx1);
            // O is stored at scale 2^(-m_run * scale2).  It is only brought to a new scale when the row's max has
            // grown by more than a factor 2^8 (so every exponent below stays <= 8) or nothing has been accumulated yet.
            const bool grow = mx > m_run + grow_by;                     // (m_run = -inf: any finite max grows it)
            const float m_new = grow ? mx : m_run;
            const float mu = (m_new == -INFINITY) ? 0.f : m_new;
            const float alpha = grow ? fast_exp2((m_run - mu) * scale2) : 1.f;      // (m_run = -inf -> 0)
            m_run = m_new;
            const float bias = -mu * scale2;
            float sum0 = 0.f, sum1 = 0.f, sum2 = 0.f, sum3 = 0.f;
            uint32_t packed[COLS / 2];
#pragma unroll
            for (int c = 0; c < COLS; c += 4) {
                const float e0 = fast_exp2(fmaf(s[c], scale2, bias)), e1 = fast_exp2(fmaf(s[c + 1], scale2, bias));
                const float e2 = fast_exp2(fmaf(s[c + 2], scale2, bias)), e3 = fast_exp2(fmaf(s[c + 3], scale2, bias));
                sum0 += e0;
                sum1 += e1;
                sum2 += e2;
                sum3 += e3;
                packed[c / 2] = pack2<T>(e0, e1);
                packed[c / 2 + 1] = pack2<T>(e2, e3);
            }
            l_run = l_run * alpha + ((sum0 + sum1) + (sum2 + sum3));

            if (warp == 0) HOGATT_TL(1, 4000 + it);
            // ---- P and O become writable once the previous tile's second MMA has finished ----
            if (it > 0) {
                ok = mbar_wait_bounded(o_done, ((uint32_t)(it - 1)) & 1u, abort_flag, a.status, STATUS_WAIT_SYNC_TIMEOUT);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
            }
            if (!d.first_of_unit && __any_sync(0xffffffffu, grow)) {
                const uint32_t o_addr = tmem + lane_base + C::COL_O + col0;
#pragma unroll 1
                for (int c = 0; c < COLS / 32; ++c) {
                    float o[32];
                    tmem_ld32(o_addr + c * 32, o);
                    tmem_wait_ld();
#pragma unroll
                    for (int k = 0; k < 32; ++k) o[k] *= alpha;
                    tmem_st32(o_addr + c * 32, o);
                }
                tmem_wait_st();
            }
            if (warp == 0) HOGATT_TL(1, 5000 + it);
            // ---- P (storage type, two per column) into tensor memory: this row's lane, this thread's columns ----
            static_assert(COLS == 64, "one 32-column store of packed probabilities per thread");
            tmem_st32(tmem + lane_base + C::COL_P + col0 / 2, *reinterpret_cast<const float(*)[32]>(&packed[0]));
            tmem_wait_st();
            // V rows at or past the fragment's true length may hold anything (spare rows of a slab, fetched as they
            // are): their probabilities are exactly zero, but 0 * NaN would poison O.  Zero them in the staged tile
            // (each thread its share of the row's bytes).
            if (d.tok0 + kDenseTile > vlen) {
                const int vs = it % C::NV;
                ok = mbar_wait_bounded(v_full + 8 * vs, ((uint32_t)(it / C::NV)) & 1u, abort_flag, a.status, STATUS_WAIT_FULL_TIMEOUT);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                if (d.tok0 + row >= vlen) {
                    unsigned char* vrow = base + C::OFF_V + vs * C::TILE_BYTES + (col0 >> 6) * C::ATOM_BYTES + row * 128 + (col0 & 63) * 2;
#pragma unroll
                    for (int c = 0; c < COLS / 8; ++c) *reinterpret_cast<int4*>(vrow + c * 16) = make_int4(0, 0, 0, 0);
                }
                fence_proxy_async_smem();      // generic-proxy writes (V rows) before the MMA's async-proxy reads
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full);
            if (warp == 0) HOGATT_TL(1, 6000 + it);

            // ---- end of this CTA's share of the unit: leave the partial result ----
            if (d.last_of_unit) {
                ok = mbar_wait_bounded(o_done, ((uint32_t)it) & 1u, abort_flag, a.status, STATUS_WAIT_SYNC_TIMEOUT);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                int first, count;
                unit_ctas(d.u, TH, N, ctas, &first, &count);
                const size_t slot = (size_t)d.u * a.parts_per_unit + (blockIdx.x - first);
                float* wo = a.ws_o + (slot * kDenseRows + row) * C::HD + col0;
                const uint32_t o_addr = tmem + lane_base + C::COL_O + col0;
#pragma unroll 1
                for (int c = 0; c < COLS / 32; ++c) {
                    float o[32];
                    tmem_ld32(o_addr + c * 32, o);
                    tmem_wait_ld();
#pragma unroll
                    for (int k = 0; k < 8; ++k)
                        *reinterpret_cast<float4*>(wo + c * 32 + k * 4) = make_float4(o[4 * k], o[4 * k + 1], o[4 * k + 2], o[4 * k + 3]);
                }
                // The row's sum is the column groups' shares added up.  Groups 1.. hand theirs to group 0 through four
                // spare tensor-memory columns (two sets, alternating: group 0 may still be reading the previous set).
                const uint32_t l_addr = tmem + lane_base + C::COL_L + (nflush & 1u) * 4;
                if (part != 0) {
                    tmem_st1(l_addr + part, l_run);
                    tmem_wait_st();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(l_ready + 8 * (warp & 3));
                } else {
                    ok = mbar_wait_bounded(l_ready + 8 * (warp & 3), nflush & 1u, abort_flag, a.status, STATUS_WAIT_SYNC_TIMEOUT);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    tc_fence_after();
                    float shares[4];
                    tmem_ld4(l_addr, shares);
                    tmem_wait_ld();
                    float total = l_run;
#pragma unroll
                    for (int k = 1; k < SPLIT; ++k) total += shares[k];
                    a.ws_m[slot * kDenseRows + row] = m_run == -INFINITY ? -INFINITY : m_run * scale2;
                    a.ws_l[slot * kDenseRows + row] = total;
                }
                ++nflush;
                tc_fence_before();
            }
        }
    }

    // ---- common exit: nobody leaves before tensor memory can be handed back ----
    tc_fence_before();
    __syncthreads();
    if (warp == kDenseSoftmaxWarps + 1) {
        tc_fence_after();
        tmem_dealloc(tmem, C::TMEM_COLS);
    }
}

}  // namespace hogatt
