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
                    const size_t row = ((size_t)table[l / a.block_size] * a.Hkv + u.hkv) * a.block_size + l % a.block_size;
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
                    const size_t row = ((size_t)table[l / a.block_size] * a.Hkv + u.hkv) * a.block_size + l % a.block_size;
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

template <class T>
__global__ void __launch_bounds__(kMergeWarps * 32) paged_merge_kernel(const __grid_constant__ PagedArgs a) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    PagedUnit u;
    if (!locate_paged_unit(a, blockIdx.x, &u)) return;
    T* const out = static_cast<T*>(a.out);
    for (int row = warp; row < kFmaRows; row += kMergeWarps) {
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
