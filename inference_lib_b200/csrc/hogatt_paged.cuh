// Paged variants of the op: `hogwild_paged_sdpa`, `hogwild_varlen_paged_sdpa`, `copy_to_blocks`.
//
// Semantics follow the reference kernels (src/kernels/kernel_v21.cuh:318-602 and :658-949,
// src/cache.cuh:6-49): the KV of worker w is a paged sequence addressed through block_table[w, :]
// (key l lives in block table[l / bs] at row l % bs of cache[NumBlocks, Hkv, bs, E]); every fragment
// index f re-reads that same sequence with its own pre-rotated query, location and length.  The
// fixed-S and the packed (varlen) layouts differ only in strides, so one kernel serves both.
//
// Work split: a unit is (group of query tokens of one worker, block of <=16 GQA heads, kv head),
// i.e. up to 16 query rows that share one paged sequence; grid = (units, splits), split s takes a
// contiguous share of the unit's 32-key tiles and always leaves a partial, the merge kernel folds
// `splits` partials per row.  The per-tile arithmetic is the FMA core of the fragment kernel.
#pragma once
#include "hogatt_device.cuh"
#include "hogatt_fma.cuh"
#include "hogatt_merge.cuh"

namespace hogatt {

struct PagedArgs {
    int F, W, Hq, Hkv, G, E, Ev;
    int S;                    // query tokens per worker (fixed layout); unused when cu_seqlens != nullptr
    int total_q;              // packed query tokens (varlen) or W * S
    int block_size, max_blocks;
    int tokens_per_group;     // query tokens per unit: max(1, 16 / G)
    int head_blocks;          // ceil(G / 16)
    int groups_bound;         // upper bound of token groups over all workers
    int splits;
    float l2scale;
    // element strides: q[f*q_f + w*q_w + s*q_s + h*q_h], out[w*o_w + s*o_s + h*o_h], loc[f*loc_f + w*loc_w + s]
    long long q_f, q_w, q_s, q_h, o_w, o_s, o_h;
    int loc_f, loc_w, len_f, len_w;
    void* out;
    const void* q;
    const int* loc;
    const int* flen;
    const void* kcache;
    const void* vcache;
    const int* block_table;
    const int* cu_seqlens;    // [W+1] or nullptr
    float* ws_o;
    float* ws_m;
    float* ws_l;
};

// Which worker and which of its token groups a global group index is.  Linear scan over workers
// (the reference does the same per CTA, src/kernels/kernel_v21.cuh:15-23).  Returns false past the end.
struct PagedUnit {
    int w, s_begin, s_end, s_base;    // query tokens [s_begin, s_end) of worker w; s_base = first token's global index offset
    int hkv, g0;
};
__device__ __forceinline__ bool locate_paged_unit(const PagedArgs& a, int x, PagedUnit* u) {
    u->hkv = x % a.Hkv;
    const int y = x / a.Hkv;
    u->g0 = (y % a.head_blocks) * 16;
    int grp = y / a.head_blocks;
    for (int w = 0; w < a.W; ++w) {
        const int start = a.cu_seqlens ? a.cu_seqlens[w] : 0;
        const int Sw = a.cu_seqlens ? a.cu_seqlens[w + 1] - start : a.S;
        const int ng = (Sw + a.tokens_per_group - 1) / a.tokens_per_group;
        if (grp < ng) {
            u->w = w;
            u->s_begin = grp * a.tokens_per_group;
            u->s_end = min(Sw, u->s_begin + a.tokens_per_group);
            u->s_base = start;
            return true;
        }
        grp -= ng;
    }
    return false;
}

// Row r of a unit: token s_begin + r / rows_per_token, head g0 + r % rows_per_token.
__device__ __forceinline__ bool paged_row(const PagedArgs& a, const PagedUnit& u, int r, int* s_abs, int* hq) {
    const int hpt = min(a.G - u.g0, 16);                  // heads of this unit per token
    const int tok = u.s_begin + r / hpt;
    const int g = u.g0 + r % hpt;
    if (tok >= u.s_end || r >= a.tokens_per_group * hpt) return false;
    *s_abs = u.s_base + tok;                              // index along the s axis of q / out / loc
    *hq = u.hkv * a.G + g;
    return true;
}

__host__ __device__ inline size_t paged_smem_bytes(int E, int Ev, int F) {
    size_t floats = (size_t)kFmaRows * E + (size_t)kFmaTile * (E + 1) + (size_t)kFmaTile * Ev +
                    (size_t)kFmaRows * kFmaTile + kFmaRows;
    return floats * sizeof(float) + ((size_t)kFmaRows + 2 * (size_t)F + 1) * sizeof(int);
}

template <class T, int EV>
__global__ void __launch_bounds__(kFmaThreads) paged_attention_kernel(const __grid_constant__ PagedArgs a) {
    constexpr int VEC = 16 / sizeof(T);
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int E = a.E, tid = threadIdx.x;
    FmaCore<EV> core;
    int* vis = reinterpret_cast<int*>(core.carve(smem_raw, E));   // [F] visible keys per fragment for this unit
    int* pre = vis + a.F;                                          // [F+1] tile prefix

    PagedUnit u;
    if (!locate_paged_unit(a, blockIdx.x, &u)) return;            // grid is an upper bound on the units
    const int split = blockIdx.y;
    const T* __restrict__ q = static_cast<const T*>(a.q);

    // visible length of every fragment for this unit: max over its rows of min(len, loc + 1)
    for (int f = tid; f < a.F; f += kFmaThreads) vis[f] = 0;
    __syncthreads();
    for (int i = tid; i < a.F * kFmaRows; i += kFmaThreads) {
        const int f = i / kFmaRows, r = i % kFmaRows;
        int s_abs, hq;
        if (paged_row(a, u, r, &s_abs, &hq)) {
            const int len = a.flen[f * a.len_f + u.w * a.len_w];
            const int loc = a.loc[(size_t)f * a.loc_f + (size_t)u.w * a.loc_w + s_abs];
            atomicMax(&vis[f], max(0, min(loc, len - 1) + 1));
        }
    }
    __syncthreads();
    if (tid == 0) {
        int acc = 0;
        for (int f = 0; f < a.F; ++f) {
            pre[f] = acc;
            acc += ceil_div(vis[f], kFmaTile);
        }
        pre[a.F] = acc;
    }
    __syncthreads();
    const int T_u = pre[a.F];
    const int t0 = (int)((int64_t)split * T_u / a.splits), t1 = (int)((int64_t)(split + 1) * T_u / a.splits);

    core.reset();
    int cur_f = -1, fscan = 0;
    for (int t = t0; t < t1; ++t) {
        while (t >= pre[fscan + 1]) ++fscan;
        const int f = fscan;
        if (f != cur_f) {
            cur_f = f;
#pragma unroll 4
            for (int idx = tid; idx < kFmaRows * E; idx += kFmaThreads) {
                const int r = idx / E, e = idx - r * E;
                int s_abs, hq;
                float val = 0.f;
                if (paged_row(a, u, r, &s_abs, &hq))
                    val = Scalar<T>::to_float(q[f * a.q_f + u.w * a.q_w + s_abs * a.q_s + hq * a.q_h + e]);
                core.Qs[idx] = val;
            }
            if (tid < kFmaRows) {
                int s_abs, hq, lim = 0;
                if (paged_row(a, u, tid, &s_abs, &hq)) {
                    const int len = a.flen[f * a.len_f + u.w * a.len_w];
                    const int loc = a.loc[(size_t)f * a.loc_f + (size_t)u.w * a.loc_w + s_abs];
                    lim = max(0, min(loc, len - 1) + 1);
                }
                core.lim_s[tid] = lim;
            }
        }
        const int tok0 = (t - pre[f]) * kFmaTile;
        const int ntok = min(kFmaTile, vis[f] - tok0);

        // ---- stage K and V rows through the block table (a row is contiguous, rows are not) ----
        {
            const int kvr = E / VEC, vvr = EV / VEC;                 // 16-byte vectors per row
            const int* table = a.block_table + (size_t)u.w * a.max_blocks;
            for (int i = tid; i < kFmaTile * kvr; i += kFmaThreads) {
                const int tok = i / kvr, c = i - tok * kvr;
                if (tok < ntok) {
                    const int l = tok0 + tok;
                    const size_t row = ((size_t)table[min(l / a.block_size, a.max_blocks - 1)] * a.Hkv + u.hkv) * a.block_size + l % a.block_size;
                    const int4 raw = __ldg(reinterpret_cast<const int4*>(static_cast<const T*>(a.kcache) + row * E) + c);
                    const T* x = reinterpret_cast<const T*>(&raw);
#pragma unroll
                    for (int k = 0; k < VEC; ++k) core.Ks[tok * (E + 1) + c * VEC + k] = Scalar<T>::to_float(x[k]);
                }
            }
            for (int i = tid; i < kFmaTile * vvr; i += kFmaThreads) {
                const int tok = i / vvr, c = i - tok * vvr;
                int4 raw = make_int4(0, 0, 0, 0);                     // rows past the tile end must be finite
                if (tok < ntok) {
                    const int l = tok0 + tok;
                    const size_t row = ((size_t)table[min(l / a.block_size, a.max_blocks - 1)] * a.Hkv + u.hkv) * a.block_size + l % a.block_size;
                    raw = __ldg(reinterpret_cast<const int4*>(static_cast<const T*>(a.vcache) + row * EV) + c);
                }
                const T* x = reinterpret_cast<const T*>(&raw);
#pragma unroll
                for (int k = 0; k < VEC; ++k) core.Vs[tok * EV + c * VEC + k] = Scalar<T>::to_float(x[k]);
            }
        }
        __syncthreads();
        core.compute(tok0, ntok, a.l2scale);
        __syncthreads();
    }
    core.flush(a.ws_o, a.ws_m, a.ws_l, (size_t)blockIdx.x * a.splits + split);
}

// ---- tensor-core paged kernel (f16 / bf16, E = Ev = 64 or 128) --------------------------------------------------
// Same units, splits, partial format and merge as paged_attention_kernel; what differs is the tile core: a tile is
// 64 keys, fetched row by row through the block table with 16-byte cp.async copies into a two-stage ring (rows past
// the tile's end are zero-filled by the copy itself), and the four warps each take 16 keys of it:
// S = Q K^T and O += P V with mma.sync m16n8k16 (query rows are the M of both), online softmax in base 2 in
// registers, P handed from the first MMA's accumulators to the second's A operand without leaving the registers.
// At the end the four warps' (O, max, sum) are folded through shared memory into the one partial the split leaves.
// Replaces the CUDA-core loops of src/kernels/kernel_v21.cuh:318-602 (paged) and :658-949 (varlen paged).
template <int HD, int NS = 2>
struct PagedMmaCfg {
    static constexpr int TILE = 64, WARPS = 4, THREADS = WARPS * 32, NSTAGE = NS;
    static constexpr int PITCH = HD * 2 + 16;                    // bytes between staged rows: 8 consecutive rows hit 8 bank groups
    static constexpr int QBYTES = kFmaRows * PITCH;
    static constexpr int OFF_LIM = QBYTES;                       // int[16]: visibility limit per query row
    static constexpr int OFF_STAGE = (QBYTES + 64 + 127) / 128 * 128;
    static constexpr int KV_BYTES = TILE * PITCH;                // K (or V) rows of one tile
    static constexpr int STAGE_BYTES = 2 * KV_BYTES;
    static constexpr int OFF_PLAN = OFF_STAGE + NSTAGE * STAGE_BYTES;       // int vis[F], pre[F + 1]
    static constexpr int FOLD_FLOATS = kFmaRows * HD + 2 * kFmaRows;        // per warp: O, max, sum
    static_assert(WARPS * FOLD_FLOATS * 4 <= NSTAGE * STAGE_BYTES, "the fold reuses the K/V ring");
};
template <int HD, int NS = 2>
__host__ __device__ inline size_t paged_mma_smem_bytes(int F) {
    return PagedMmaCfg<HD, NS>::OFF_PLAN + ((size_t)2 * F + 1) * sizeof(int);
}

__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, bool real) {
    const int n = real ? 16 : 0;                                  // 0 source bytes: the 16 destination bytes become zero
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <class T, int HD, int NS = 2>
__global__ void __launch_bounds__(PagedMmaCfg<HD, NS>::THREADS) paged_mma_kernel(const __grid_constant__ PagedArgs a) {
    using C = PagedMmaCfg<HD, NS>;
    constexpr int KSTEPS = HD / 16, NT_O = HD / 8, CPR = HD / 8;     // k-steps of QK^T, n-tiles of O, 16-byte chunks per row
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    unsigned char* qtile = smem_raw;
    int* lim_s = reinterpret_cast<int*>(smem_raw + C::OFF_LIM);
    unsigned char* stages = smem_raw + C::OFF_STAGE;
    int* vis = reinterpret_cast<int*>(smem_raw + C::OFF_PLAN);
    int* pre = vis + a.F;

    // Launched with programmatic stream serialization: wait for the stream's earlier work before anything is read,
    // then let the merge kernel take its place on the SMs (it waits for this whole grid itself).
    pdl_wait();
    pdl_trigger();
    PagedUnit u;
    if (!locate_paged_unit(a, blockIdx.x, &u)) return;            // (uniform over the CTA)
    const int split = blockIdx.y;
    const T* __restrict__ q = static_cast<const T*>(a.q);
    const T* __restrict__ kc = static_cast<const T*>(a.kcache);
    const T* __restrict__ vc = static_cast<const T*>(a.vcache);
    const int* __restrict__ table = a.block_table + (size_t)u.w * a.max_blocks;

    // visible length of every fragment for this unit: max over its rows of min(len, loc + 1)
    for (int f = tid; f < a.F; f += C::THREADS) vis[f] = 0;
    __syncthreads();
    for (int i = tid; i < a.F * kFmaRows; i += C::THREADS) {
        const int f = i / kFmaRows, r = i % kFmaRows;
        int s_abs, hq;
        if (paged_row(a, u, r, &s_abs, &hq)) {
            const int len = a.flen[f * a.len_f + u.w * a.len_w];
            const int loc = a.loc[(size_t)f * a.loc_f + (size_t)u.w * a.loc_w + s_abs];
            atomicMax(&vis[f], max(0, min(loc, len - 1) + 1));
        }
    }
    __syncthreads();
    if (tid == 0) {
        int acc = 0;
        for (int f = 0; f < a.F; ++f) {
            pre[f] = acc;
            acc += ceil_div(vis[f], C::TILE);
        }
        pre[a.F] = acc;
    }
    __syncthreads();
    const int T_u = pre[a.F];
    const int t0 = (int)((int64_t)split * T_u / a.splits), t1 = (int)((int64_t)(split + 1) * T_u / a.splits);

    // One tile's rows into a stage.  The copies are dealt as pass k = 0 .. NP-1 of RP rows, a thread takes chunk
    // lane % CPR of row (tid / CPR) + k * RP; a warp therefore touches 16 distinct rows of the tile, and lane j < 16
    // looks up row j's place in the cache (one division and one block-table load per thread and tile) for the others.
    auto fetch = [&](int t, int stage, int fhint) {
        constexpr int RP = C::THREADS / CPR, NP = C::TILE / RP, RW = 32 / CPR;
        int f = fhint;
        while (t >= pre[f + 1]) ++f;
        const int tok0 = (t - pre[f]) * C::TILE;
        const int ntok = min(C::TILE, vis[f] - tok0);
        const uint32_t base = smem_u32(stages + stage * C::STAGE_BYTES);
        long long mine = 0;
        {
            const int j = lane & 15;
            const int tok = warp * RW + (j % RW) + (j / RW) * RP;
            const int l = tok0 + (tok < ntok ? tok : 0);
            const int blk = l / a.block_size;
            // (a length beyond the block table is the caller's error; the lookup stays inside the table regardless)
            mine = ((long long)table[min(blk, a.max_blocks - 1)] * a.Hkv + u.hkv) * a.block_size + (l - blk * a.block_size);
        }
        const int c = lane % CPR, sub = lane / CPR;
#pragma unroll
        for (int k = 0; k < NP; ++k) {
            const long long row = __shfl_sync(0xffffffffu, mine, k * RW + sub);
            const int tok = warp * RW + sub + k * RP;
            const bool real = tok < ntok;
            cp_async_16(base + tok * C::PITCH + c * 16, kc + row * HD + c * 8, real);
            cp_async_16(base + C::KV_BYTES + tok * C::PITCH + c * 16, vc + row * HD + c * 8, real);
        }
        cp_async_commit();
    };

    float o[NT_O][4];
#pragma unroll
    for (int n = 0; n < NT_O; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;    // rows lane / 4 and lane / 4 + 8
    uint32_t qf[KSTEPS][4];
    int lim0 = 0, lim1 = 0, cur_f = -1, fscan = 0;
    // the ring: tiles t .. t + NSTAGE - 2 are in flight while tile t is used (one commit group per tile, empty past the end)
#pragma unroll
    for (int k = 0; k < C::NSTAGE - 1; ++k) {
        if (t0 + k < t1) fetch(t0 + k, k, 0);
        else cp_async_commit();
    }
#pragma unroll 1
    for (int t = t0, it = 0; t < t1; ++t, ++it) {
        while (t >= pre[fscan + 1]) ++fscan;
        const int f = fscan;
        cp_async_wait<C::NSTAGE - 2>();                             // this thread's copies of tile t have landed
        __syncthreads();                                            // everyone's have, and everyone has left tile t - 1
        if (t + C::NSTAGE - 1 < t1) fetch(t + C::NSTAGE - 1, (it + C::NSTAGE - 1) % C::NSTAGE, fscan);   // into tile t - 1's stage
        else cp_async_commit();
        if (f != cur_f) {
            // this fragment's query rows (already rotated) and their limits; the query tile is only read right after
            // it is written (the A fragments stay in registers), and a barrier has passed since
            cur_f = f;
            for (int i = tid; i < kFmaRows * CPR; i += C::THREADS) {
                const int r = i / CPR, c = i - r * CPR;
                int s_abs, hq;
                uint4 val = make_uint4(0u, 0u, 0u, 0u);
                if (paged_row(a, u, r, &s_abs, &hq))
                    val = *reinterpret_cast<const uint4*>(q + f * a.q_f + u.w * a.q_w + s_abs * a.q_s + hq * a.q_h + c * 8);
                *reinterpret_cast<uint4*>(qtile + r * C::PITCH + c * 16) = val;
            }
            if (tid < kFmaRows) {
                int s_abs, hq, lim = 0;
                if (paged_row(a, u, tid, &s_abs, &hq)) {
                    const int len = a.flen[f * a.len_f + u.w * a.len_w];
                    const int loc = a.loc[(size_t)f * a.loc_f + (size_t)u.w * a.loc_w + s_abs];
                    lim = max(0, min(loc, len - 1) + 1);
                }
                lim_s[tid] = lim;
            }
            __syncthreads();
            const uint32_t qaddr = smem_u32(qtile) + ((lane & 7) + ((lane >> 3) & 1) * 8) * C::PITCH + (lane >> 4) * 16;
#pragma unroll
            for (int kk = 0; kk < KSTEPS; ++kk) ldmatrix_x4(qaddr + kk * 32, qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3]);
            lim0 = lim_s[lane >> 2];
            lim1 = lim_s[(lane >> 2) + 8];
        }

        const int tok0 = (t - pre[f]) * C::TILE;
        const uint32_t sk = smem_u32(stages + (it % C::NSTAGE) * C::STAGE_BYTES), sv = sk + C::KV_BYTES;
        const int kw0 = warp * 16;                                  // this warp's 16 keys of the tile
        float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        {
            const uint32_t kaddr = sk + (kw0 + (lane & 7) + ((lane >> 4) & 1) * 8) * C::PITCH + ((lane >> 3) & 1) * 16;
#pragma unroll
            for (int kk = 0; kk < KSTEPS; ++kk) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4(kaddr + kk * 32, b0, b1, b2, b3);
                mma_16816<T>(s[0], qf[kk], b0, b1);
                mma_16816<T>(s[1], qf[kk], b2, b3);
            }
        }
        // mask, online softmax (base 2); a key is visible to a row iff its index is below the row's limit
        const int key0 = tok0 + kw0 + (lane & 3) * 2;
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int key = key0 + j * 8 + i;
                s[j][i] = key < lim0 ? s[j][i] * a.l2scale : -INFINITY;
                s[j][2 + i] = key < lim1 ? s[j][2 + i] * a.l2scale : -INFINITY;
                mx0 = fmaxf(mx0, s[j][i]);
                mx1 = fmaxf(mx1, s[j][2 + i]);
            }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
        const float mu0 = n0 == -INFINITY ? 0.f : n0, mu1 = n1 == -INFINITY ? 0.f : n1;
        const float al0 = exp2f(m0 - mu0), al1 = exp2f(m1 - mu1);   // (-inf -> 0)
        m0 = n0;
        m1 = n1;
        // a row's maximum settles after a few tiles: the accumulators are rescaled only when some row's has grown
        const bool grew = __any_sync(0xffffffffu, al0 != 1.f || al1 != 1.f);
        float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                s[j][i] = exp2f(s[j][i] - mu0);
                s[j][2 + i] = exp2f(s[j][2 + i] - mu1);
                ps0 += s[j][i];
                ps1 += s[j][2 + i];
            }
        l0 = l0 * al0 + ps0;                                        // per-thread shares; the four lanes of a row add up at the end
        l1 = l1 * al1 + ps1;
        uint32_t pa[4];
        pa[0] = pack2<T>(s[0][0], s[0][1]);
        pa[1] = pack2<T>(s[0][2], s[0][3]);
        pa[2] = pack2<T>(s[1][0], s[1][1]);
        pa[3] = pack2<T>(s[1][2], s[1][3]);
        {
            const uint32_t vaddr = sv + (kw0 + (lane & 7) + ((lane >> 3) & 1) * 8) * C::PITCH + ((lane >> 4) & 1) * 16;
#pragma unroll
            for (int n = 0; n < NT_O; n += 2) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4_trans(vaddr + n * 16, b0, b1, b2, b3);
                if (grew) {
                    o[n][0] *= al0; o[n][1] *= al0; o[n][2] *= al1; o[n][3] *= al1;
                    o[n + 1][0] *= al0; o[n + 1][1] *= al0; o[n + 1][2] *= al1; o[n + 1][3] *= al1;
                }
                mma_16816<T>(o[n], pa, b0, b1);
                mma_16816<T>(o[n + 1], pa, b2, b3);
            }
        }
    }
    __syncthreads();                                                // every warp has left the last tile: the ring is free

    // ---- fold the four warps' results into the split's partial -------------------------------------------------
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    float* fold = reinterpret_cast<float*>(stages) + warp * C::FOLD_FLOATS;       // [16][HD] O, [16] max, [16] sum
    {
        const int r0 = lane >> 2, c0 = (lane & 3) * 2;
#pragma unroll
        for (int n = 0; n < NT_O; ++n) {
            *reinterpret_cast<float2*>(fold + r0 * HD + n * 8 + c0) = make_float2(o[n][0], o[n][1]);
            *reinterpret_cast<float2*>(fold + (r0 + 8) * HD + n * 8 + c0) = make_float2(o[n][2], o[n][3]);
        }
        if ((lane & 3) == 0) {
            fold[kFmaRows * HD + r0] = m0;
            fold[kFmaRows * HD + r0 + 8] = m1;
            fold[kFmaRows * HD + kFmaRows + r0] = l0;
            fold[kFmaRows * HD + kFmaRows + r0 + 8] = l1;
        }
    }
    __syncthreads();
    const float* all = reinterpret_cast<const float*>(stages);
    const size_t slot = (size_t)blockIdx.x * a.splits + split;
    for (int i = tid; i < kFmaRows * (HD / 4); i += C::THREADS) {
        const int r = i / (HD / 4), c = (i - r * (HD / 4)) * 4;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < C::WARPS; ++w) M = fmaxf(M, all[w * C::FOLD_FLOATS + kFmaRows * HD + r]);
        const float mu = M == -INFINITY ? 0.f : M;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        float L = 0.f;
#pragma unroll
        for (int w = 0; w < C::WARPS; ++w) {
            const float* fw = all + w * C::FOLD_FLOATS;
            const float wgt = exp2f(fw[kFmaRows * HD + r] - mu);    // a warp that saw nothing: 2^-inf = 0, its O is zero too
            const float4 x = *reinterpret_cast<const float4*>(fw + r * HD + c);
            acc.x = fmaf(x.x, wgt, acc.x);
            acc.y = fmaf(x.y, wgt, acc.y);
            acc.z = fmaf(x.z, wgt, acc.z);
            acc.w = fmaf(x.w, wgt, acc.w);
            L = fmaf(fw[kFmaRows * HD + kFmaRows + r], wgt, L);
        }
        *reinterpret_cast<float4*>(a.ws_o + (slot * kFmaRows + r) * HD + c) = acc;
        if (c == 0) {
            a.ws_m[slot * kFmaRows + r] = M;
            a.ws_l[slot * kFmaRows + r] = L;
        }
    }
}

template <class T>
__global__ void __launch_bounds__(kMergeWarps * 32) paged_merge_kernel(const __grid_constant__ PagedArgs a) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    pdl_wait();                                                    // (returns at once after an ordinary launch)
    PagedUnit u;
    if (!locate_paged_unit(a, blockIdx.x, &u)) return;
    T* const out = static_cast<T*>(a.out);
    // grid (units, row groups): one warp per output row where the grid allows, so that a row's partials are one round trip
    for (int row = blockIdx.y * kMergeWarps + warp; row < kFmaRows; row += gridDim.y * kMergeWarps) {
        int s_abs, hq;
        if (!paged_row(a, u, row, &s_abs, &hq)) continue;
        const int splits = a.splits;
#pragma unroll 1
        for (int e0 = 0; e0 < a.Ev; e0 += 128)
            merge_partials_rows<T, 1, 24>(a.ws_o, a.ws_m, a.ws_l, (size_t)blockIdx.x * a.splits, kFmaRows, a.Ev, row, splits,
                                      [splits]() { return splits; }, &out, 1,
                                      (size_t)(u.w * a.o_w + s_abs * a.o_s + hq * a.o_h), lane, e0);
    }
}

// Append S_new rows per (batch, kv head) to the paged caches at positions seq_lengths[b] + t.
// One 16-byte vector per thread; replaces copy_to_blocks_kernel (src/cache.cuh:6-49), where every
// thread of a (S_new x head-size) block copies a whole row element by element.
template <class T>
__global__ void __launch_bounds__(256) copy_to_blocks_kernel(const T* __restrict__ k_states, const T* __restrict__ v_states,
                                                             T* __restrict__ k_cache, T* __restrict__ v_cache,
                                                             const int* __restrict__ block_table,
                                                             const int* __restrict__ seq_lengths, int B, int Hkv,
                                                             int S_new, int E, int Ev, int block_size, int max_blocks) {
    constexpr int VEC = 16 / sizeof(T);
    const int kvr = E / VEC, vvr = Ev / VEC, per_row = kvr + vvr;
    const int64_t total = (int64_t)B * Hkv * S_new * per_row;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int c = (int)(i % per_row);
        int64_t r = i / per_row;
        const int t = (int)(r % S_new);
        r /= S_new;
        const int h = (int)(r % Hkv);
        const int b = (int)(r / Hkv);
        const int pos = seq_lengths[b] + t;
        const size_t blk = (size_t)block_table[(size_t)b * max_blocks + pos / block_size];
        const size_t dst_row = (blk * Hkv + h) * block_size + pos % block_size;
        const size_t src_row = ((size_t)b * Hkv + h) * S_new + t;
        if (c < kvr)
            reinterpret_cast<int4*>(k_cache + dst_row * E)[c] = __ldg(reinterpret_cast<const int4*>(k_states + src_row * E) + c);
        else
            reinterpret_cast<int4*>(v_cache + dst_row * Ev)[c - kvr] =
                __ldg(reinterpret_cast<const int4*>(v_states + src_row * Ev) + (c - kvr));
    }
}

}  // namespace hogatt
