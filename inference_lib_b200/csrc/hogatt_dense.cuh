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
//     thread; S (two buffers) and O live in tensor memory.  Four softmax warps -- one thread per query row -- pull
//     S out of tensor memory (tcgen05.ld), mask, exponentiate, write P as bf16/f16 into shared memory for the
//     second MMA, and keep the running max and sum in registers.  O is rescaled in tensor memory only when a row's
//     max has grown by more than 2^8 since the scale it is stored at (then exp2 arguments stay below 8 and
//     nothing overflows); the stored scale travels with the partial result, so the merge is exact.
//
// Warp roles (192 threads): warps 0-3 softmax (warp w owns tensor-memory lanes 32w..32w+31), warp 4 issues the
// K/V copies, warp 5 allocates tensor memory, issues the Q copies and every MMA.  Every wait is bounded.
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
constexpr int kDenseThreads = 192;

struct alignas(64) DenseMaps {
    CUtensorMap q;                          // [F, W, Hkv, G*S, E] view of the rotated queries
    CUtensorMap k[kDenseMaxFragments];      // [Hkv, rows, E] per fragment
    CUtensorMap v[kDenseMaxFragments];      // [Hkv, rows, Ev]
};

struct DenseCfg {
    static constexpr int HD = 128;
    static constexpr int ATOM_BYTES = 128 * 128;            // [128 rows][64 16-bit columns], rows of 128 bytes, swizzled
    static constexpr int TILE_BYTES = 2 * ATOM_BYTES;       // a 128 x 128 operand tile: two column halves
    static constexpr int NK = 3, NV = 2;                    // K ring, V ring
    static constexpr int OFF_Q = 0;
    static constexpr int OFF_P = OFF_Q + TILE_BYTES;
    static constexpr int OFF_K = OFF_P + TILE_BYTES;
    static constexpr int OFF_V = OFF_K + NK * TILE_BYTES;
    static constexpr int OFF_BAR = OFF_V + NV * TILE_BYTES;                 // 224 KiB of tiles
    // barriers: q_full, k_full[NK], k_empty[NK], v_full[NV], v_empty[NV], s_full[2], s_free[2], p_full, o_done
    static constexpr int NBAR = 1 + 2 * NK + 2 * NV + 2 + 2 + 1 + 1;
    static constexpr int OFF_MISC = OFF_BAR + NBAR * 8;                     // tmem base, abort flag
    static constexpr int OFF_PLAN = OFF_MISC + 16;                          // vis[F], pre[F + 1]
    static constexpr int TMEM_COLS = 512;
    static constexpr int COL_O = 0, COL_S0 = 128, COL_S1 = 256;
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
                   o_done = p_full + 8;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base + C::OFF_MISC);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(base + C::OFF_MISC + 8);
    int* vis = reinterpret_cast<int*>(base + C::OFF_PLAN);
    int* pre = vis + a.F;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

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
            mbar_init(s_free + 8 * s, 4);      // one arrival per softmax warp
        }
        mbar_init(p_full, 4);
        mbar_init(o_done, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_proxy_async_smem();
    }
    if (warp == 5) tmem_alloc(smem_u32(tmem_slot), C::TMEM_COLS);
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
    const int ctas = effective_ctas(N, gridDim.x);
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

    if (warp == 4) {
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
    } else if (warp == 5) {
        // ============================== Q copies and every MMA ==============================
        if (lane == 0) {
            constexpr uint32_t IDESC_S = umma_idesc<T>(false, kDenseRows, kDenseTile);
            constexpr uint32_t IDESC_O = umma_idesc<T>(true, kDenseRows, C::HD);
            const uint32_t q_smem = sbase + C::OFF_Q, p_smem = sbase + C::OFF_P;
            uint32_t q_phase = 0;
            auto load_q = [&](const DenseTile& d) {
                const int r0 = d.rb * kDenseRows;
                mbar_arrive_expect_tx(q_full, C::TILE_BYTES);
                tma_load_5d(q_smem, &maps.q, 0, r0 % GS, d.hkv, r0 / GS, d.f, q_full);
                tma_load_5d(q_smem + C::ATOM_BYTES, &maps.q, 64, r0 % GS, d.hkv, r0 / GS, d.f, q_full);
            };
            // S_it = Q K^T into S buffer it & 1 (K ring stage it % NK); the stage is handed back when the MMAs are done
            auto issue_s = [&](int it) -> bool {
                const int ks = it % C::NK, sb = it & 1;
                if (!mbar_wait_bounded(k_full + 8 * ks, ((uint32_t)(it / C::NK)) & 1u, abort_flag, a.status, STATUS_WAIT_FULL_TIMEOUT))
                    return false;
                if (!mbar_wait_bounded(s_free + 8 * sb, (((uint32_t)(it >> 1)) & 1u) ^ 1u, abort_flag, a.status, STATUS_WAIT_SYNC_TIMEOUT))
                    return false;
                tc_fence_after();
                const uint32_t k_smem = sbase + C::OFF_K + ks * C::TILE_BYTES;
                const uint32_t d_tmem = tmem + (sb ? C::COL_S1 : C::COL_S0);
#pragma unroll
                for (int kk = 0; kk < C::HD / 16; ++kk) {
                    const uint32_t off = (kk >> 2) * C::ATOM_BYTES + (kk & 3) * 32;
                    tc_mma(d_tmem, umma_desc(q_smem + off, 16, 1024), umma_desc(k_smem + off, 16, 1024), IDESC_S, kk > 0);
                }
                tc_commit(s_full + 8 * sb);
                tc_commit(k_empty + 8 * ks);
                return true;
            };

            DenseWalk walk(vis, pre, a.F, a.Hkv, t0, t1);
            bool ok = true;
            DenseTile cur, nxt;
            bool have_next = !walk.done();
            if (have_next) {
                nxt = walk.next();
                load_q(nxt);
                ok = mbar_wait_bounded(q_full, q_phase, abort_flag, a.status, STATUS_WAIT_FULL_TIMEOUT);
                q_phase ^= 1u;
                ok = ok && issue_s(0);
            }
            for (int it = 0; have_next && ok; ++it) {
                cur = nxt;
                have_next = !walk.done();
                bool reload = false;
                if (have_next) {
                    nxt = walk.next();
                    reload = nxt.new_segment;
                    if (!reload) {
                        ok = issue_s(it + 1);
                        if (!ok) break;
                    } else {
                        // the query tile changes: S_it must be finished with the old one before it is overwritten
                        ok = mbar_wait_bounded(s_full + 8 * (it & 1), ((uint32_t)(it >> 1)) & 1u, abort_flag, a.status,
                                               STATUS_WAIT_SYNC_TIMEOUT);
                        if (!ok) break;
                        load_q(nxt);
                    }
                }
                // O (+)= P_it V_it
                const int vs = it % C::NV;
                ok = mbar_wait_bounded(p_full, ((uint32_t)it) & 1u, abort_flag, a.status, STATUS_WAIT_SYNC_TIMEOUT) &&
                     mbar_wait_bounded(v_full + 8 * vs, ((uint32_t)(it / C::NV)) & 1u, abort_flag, a.status, STATUS_WAIT_FULL_TIMEOUT);
                if (!ok) break;
                tc_fence_after();
                const uint32_t v_smem = sbase + C::OFF_V + vs * C::TILE_BYTES;
#pragma unroll
                for (int kk = 0; kk < kDenseTile / 16; ++kk) {
                    const uint32_t aoff = (kk >> 2) * C::ATOM_BYTES + (kk & 3) * 32;
                    // V is [key][Ev]: Ev (the MMA's N) is contiguous -> MN-major; 16 keys per step = two 8-key swizzle atoms
                    tc_mma(tmem + C::COL_O, umma_desc(p_smem + aoff, 16, 1024), umma_desc(v_smem + kk * 2048, C::ATOM_BYTES, 1024),
                           IDESC_O, (kk > 0 || !cur.first_of_unit) ? 1u : 0u);
                }
                tc_commit(o_done);
                tc_commit(v_empty + 8 * vs);
                if (reload) {
                    ok = mbar_wait_bounded(q_full, q_phase, abort_flag, a.status, STATUS_WAIT_FULL_TIMEOUT);
                    q_phase ^= 1u;
                    ok = ok && issue_s(it + 1);
                }
            }
        }
    } else {
        // ============================== softmax: one thread per query row ==============================
        const int row = tid;                                   // row of the block == tensor-memory lane
        const uint32_t lane_base = ((uint32_t)(warp * 32)) << 16;
        const uint32_t p_row = sbase + C::OFF_P + row * 128;   // this row's 128 bytes inside a [128][64] swizzled atom
        float m_run = -INFINITY, l_run = 0.f;
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
            ok = mbar_wait_bounded(s_full + 8 * sb, ((uint32_t)(it >> 1)) & 1u, abort_flag, a.status, STATUS_WAIT_FULL_TIMEOUT);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            float s[128];
            {
                const uint32_t src = tmem + lane_base + (sb ? C::COL_S1 : C::COL_S0);
#pragma unroll
                for (int c = 0; c < 4; ++c) tmem_ld32(src + c * 32, *reinterpret_cast<float(*)[32]>(&s[c * 32]));
                tmem_wait_ld();
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(s_free + 8 * sb);        // the next S MMA may overwrite this buffer

            // ---- scale, mask, tile max ----
            const int nvis = lim - d.tok0;                      // keys of this tile the row sees: [0, nvis)
            float mx = -INFINITY;
            if (nvis >= kDenseTile) {
#pragma unroll
                for (int c = 0; c < 128; ++c) {
                    s[c] *= a.l2scale;
                    mx = fmaxf(mx, s[c]);
                }
            } else {
#pragma unroll
                for (int c = 0; c < 128; ++c) {
                    s[c] = c < nvis ? s[c] * a.l2scale : -INFINITY;
                    mx = fmaxf(mx, s[c]);
                }
            }
            // O is stored at scale 2^-m_run.  It is only brought to a new scale when the row's max has grown by
            // more than 8 (then every exponent below stays <= 8) or when nothing has been accumulated yet.
            const bool grow = mx > m_run + 8.f || (m_run == -INFINITY && mx > -INFINITY);
            const float m_new = grow ? mx : m_run;
            const float mu = (m_new == -INFINITY) ? 0.f : m_new;
            const float alpha = grow ? exp2f(m_run - mu) : 1.f;     // (m_run = -inf -> 0)
            m_run = m_new;
            float sum = 0.f;
#pragma unroll
            for (int c = 0; c < 128; ++c) {
                s[c] = exp2f(s[c] - mu);
                sum += s[c];
            }
            l_run = l_run * alpha + sum;

            // ---- P and O become writable once the previous tile's second MMA has finished ----
            if (it > 0) {
                ok = mbar_wait_bounded(o_done, ((uint32_t)(it - 1)) & 1u, abort_flag, a.status, STATUS_WAIT_SYNC_TIMEOUT);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
            }
            if (!d.first_of_unit && __any_sync(0xffffffffu, grow)) {
                const uint32_t o_addr = tmem + lane_base + C::COL_O;
#pragma unroll 1
                for (int c = 0; c < 4; ++c) {
                    float o[32];
                    tmem_ld32(o_addr + c * 32, o);
                    tmem_wait_ld();
#pragma unroll
                    for (int k = 0; k < 32; ++k) o[k] *= alpha;
                    tmem_st32(o_addr + c * 32, o);
                }
                tmem_wait_st();
            }
            // ---- P (storage type) into shared memory, 128-byte swizzle: 16-byte chunk c of row r sits at c ^ (r & 7) ----
#pragma unroll
            for (int c = 0; c < 16; ++c) {
                uint4 v;
                v.x = pack2<T>(s[c * 8 + 0], s[c * 8 + 1]);
                v.y = pack2<T>(s[c * 8 + 2], s[c * 8 + 3]);
                v.z = pack2<T>(s[c * 8 + 4], s[c * 8 + 5]);
                v.w = pack2<T>(s[c * 8 + 6], s[c * 8 + 7]);
                const uint32_t dst = p_row + (c >> 3) * C::ATOM_BYTES + (((c & 7) ^ (row & 7)) << 4);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
            }
            // V rows at or past the fragment's true length may hold anything (spare rows of a slab, fetched as they
            // are): their probabilities are exactly zero, but 0 * NaN would poison O.  Zero them in the staged tile.
            if (d.tok0 + kDenseTile > vlen) {
                const int vs = it % C::NV;
                ok = mbar_wait_bounded(v_full + 8 * vs, ((uint32_t)(it / C::NV)) & 1u, abort_flag, a.status, STATUS_WAIT_FULL_TIMEOUT);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                if (d.tok0 + row >= vlen) {
                    unsigned char* vrow = base + C::OFF_V + vs * C::TILE_BYTES + row * 128;
#pragma unroll
                    for (int h = 0; h < 2; ++h)
#pragma unroll
                        for (int c = 0; c < 8; ++c) *reinterpret_cast<int4*>(vrow + h * C::ATOM_BYTES + c * 16) = make_int4(0, 0, 0, 0);
                }
            }
            fence_proxy_async_smem();          // generic-proxy writes (P, V rows) before the MMA's async-proxy reads
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full);

            // ---- end of this CTA's share of the unit: leave the partial result ----
            if (d.last_of_unit) {
                ok = mbar_wait_bounded(o_done, ((uint32_t)it) & 1u, abort_flag, a.status, STATUS_WAIT_SYNC_TIMEOUT);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                int first, count;
                unit_ctas(d.u, TH, N, ctas, &first, &count);
                const size_t slot = (size_t)d.u * a.parts_per_unit + (blockIdx.x - first);
                float* wo = a.ws_o + (slot * kDenseRows + row) * C::HD;
                const uint32_t o_addr = tmem + lane_base + C::COL_O;
#pragma unroll 1
                for (int c = 0; c < 4; ++c) {
                    float o[32];
                    tmem_ld32(o_addr + c * 32, o);
                    tmem_wait_ld();
#pragma unroll
                    for (int k = 0; k < 8; ++k)
                        *reinterpret_cast<float4*>(wo + c * 32 + k * 4) = make_float4(o[4 * k], o[4 * k + 1], o[4 * k + 2], o[4 * k + 3]);
                }
                a.ws_m[slot * kDenseRows + row] = m_run;
                a.ws_l[slot * kDenseRows + row] = l_run;
                tc_fence_before();
            }
        }
    }

    // ---- common exit: nobody leaves before tensor memory can be handed back ----
    tc_fence_before();
    __syncthreads();
    if (warp == 5) {
        tc_fence_after();
        tmem_dealloc(tmem, C::TMEM_COLS);
    }
}

}  // namespace hogatt
