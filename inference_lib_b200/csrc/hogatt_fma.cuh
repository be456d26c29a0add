// CUDA-core (FMA) fragment attention: any storage type (fp32 / fp16 / bf16), any qk head size
// up to 256, v head size in {32, 64, 128, 256}.  This is the path for shapes whose query tile is
// too thin or too oddly sized for the tensor-core kernel (and for fp32, where tensor cores would
// mean tf32 rounding); it uses the same persistent split-K decomposition, workspace format and
// merge step as the tensor-core kernel.
//
// Same math as the reference kernel (src/kernels/kernel_v21.cuh:95-203: per fragment, dot
// products in fp32, online softmax in base 2, fp32 weighted sum), different organisation: a CTA
// keeps 16 query rows of one kv head (all workers and GQA heads share each K/V tile) instead of
// one (worker, token) per CTA.
#pragma once
#include "hogatt_device.cuh"

namespace hogatt {

constexpr int kFmaThreads = 256;
constexpr int kFmaRows = 16;      // query rows per CTA
constexpr int kFmaTile = 32;      // keys per tile (one per lane)

__host__ __device__ inline size_t fma_smem_bytes(int E, int Ev, int F) {
    size_t floats = (size_t)kFmaRows * E + (size_t)kFmaTile * (E + 1) + (size_t)kFmaTile * Ev +
                    (size_t)kFmaRows * kFmaTile + kFmaRows;
    size_t ints = kFmaRows + (size_t)F + (size_t)F + 1;
    return floats * sizeof(float) + ints * sizeof(int);
}

// The per-tile arithmetic of the FMA path, shared by the fragment kernel and the paged kernels:
// 16 query rows (fp32 in shared memory) against up to 32 staged keys/values (fp32 in shared memory).
// Warp w owns the softmax statistics of rows w and w + 8; every thread owns RPT outputs of one column.
template <int EV>
struct FmaCore {
    static constexpr int TPC = kFmaThreads / EV;      // threads per output column
    static constexpr int RPT = kFmaRows / TPC;        // rows per thread in the PV step
    static_assert(TPC >= 1 && RPT >= 1 && RPT * TPC == kFmaRows, "EV must be 32, 64, 128 or 256");

    float *Qs, *Ks, *Vs, *Ps, *alpha_s;
    int* lim_s;
    int E, lane, warp, out_e, out_r0;
    float m0, m1, l0s, l1s;
    float acc[RPT];

    // carve [16][E] Q, [32][E+1] K, [32][EV] V, [16][32] P, [16] alpha, [16] limits; returns the end
    __device__ __forceinline__ unsigned char* carve(unsigned char* base, int E_) {
        E = E_;
        Qs = reinterpret_cast<float*>(base);
        Ks = Qs + kFmaRows * E;
        Vs = Ks + kFmaTile * (E + 1);
        Ps = Vs + kFmaTile * EV;
        alpha_s = Ps + kFmaRows * kFmaTile;
        lim_s = reinterpret_cast<int*>(alpha_s + kFmaRows);
        lane = threadIdx.x & 31;
        warp = threadIdx.x >> 5;
        out_e = threadIdx.x % EV;
        out_r0 = (threadIdx.x / EV) * RPT;
        return reinterpret_cast<unsigned char*>(lim_s + kFmaRows);
    }
    __device__ __forceinline__ void reset() {
        m0 = m1 = -INFINITY;
        l0s = l1s = 0.f;
#pragma unroll
        for (int r = 0; r < RPT; ++r) acc[r] = 0.f;
    }
    // Keys tok0 .. tok0+ntok-1 are staged (V rows past ntok zeroed) and the CTA has synchronised.
    // Key `k` is visible to row r iff k < lim_s[r].  Ends before the trailing __syncthreads().
    __device__ __forceinline__ void compute(int tok0, int ntok, float l2scale) {
        {
            float s0 = 0.f, s1 = 0.f;
            if (lane < ntok) {
                const float* kr = Ks + lane * (E + 1);
                const float* qa = Qs + warp * E;
                const float* qb = Qs + (warp + 8) * E;
                for (int e = 0; e < E; ++e) {
                    const float kv = kr[e];
                    s0 = fmaf(qa[e], kv, s0);
                    s1 = fmaf(qb[e], kv, s1);
                }
            }
            const int key = tok0 + lane;
            s0 = (lane < ntok && key < lim_s[warp]) ? s0 * l2scale : -INFINITY;
            s1 = (lane < ntok && key < lim_s[warp + 8]) ? s1 * l2scale : -INFINITY;
            float x0 = s0, x1 = s1;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                x0 = fmaxf(x0, __shfl_xor_sync(0xffffffffu, x0, o));
                x1 = fmaxf(x1, __shfl_xor_sync(0xffffffffu, x1, o));
            }
            const float n0 = fmaxf(m0, x0), n1 = fmaxf(m1, x1);
            const float b0 = (n0 == -INFINITY) ? 0.f : n0, b1 = (n1 == -INFINITY) ? 0.f : n1;
            const float a0 = exp2f(m0 - b0), a1 = exp2f(m1 - b1);
            const float p0 = exp2f(s0 - b0), p1 = exp2f(s1 - b1);
            float y0 = p0, y1 = p1;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                y0 += __shfl_xor_sync(0xffffffffu, y0, o);
                y1 += __shfl_xor_sync(0xffffffffu, y1, o);
            }
            l0s = l0s * a0 + y0;
            l1s = l1s * a1 + y1;
            m0 = n0;
            m1 = n1;
            Ps[warp * kFmaTile + lane] = p0;
            Ps[(warp + 8) * kFmaTile + lane] = p1;
            if (lane == 0) {
                alpha_s[warp] = a0;
                alpha_s[warp + 8] = a1;
            }
        }
        __syncthreads();
#pragma unroll
        for (int r = 0; r < RPT; ++r) {
            const int row = out_r0 + r;
            float v = acc[r] * alpha_s[row];
            const float* pr = Ps + row * kFmaTile;
#pragma unroll 8
            for (int k = 0; k < kFmaTile; ++k) v = fmaf(pr[k], Vs[k * EV + out_e], v);
            acc[r] = v;
        }
    }
    // unnormalised partial -> workspace slot
    __device__ __forceinline__ void flush(float* ws_o, float* ws_m, float* ws_l, size_t slot) const {
#pragma unroll
        for (int r = 0; r < RPT; ++r) ws_o[(slot * kFmaRows + out_r0 + r) * EV + out_e] = acc[r];
        if (lane == 0) {
            ws_m[slot * kFmaRows + warp] = m0;
            ws_m[slot * kFmaRows + warp + 8] = m1;
            ws_l[slot * kFmaRows + warp] = l0s;
            ws_l[slot * kFmaRows + warp + 8] = l1s;
        }
    }
};

template <class T, int EV>
__global__ void __launch_bounds__(kFmaThreads) fma_attention_kernel(const __grid_constant__ KernelArgs a) {
    constexpr int VEC = 16 / sizeof(T);
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int E = a.E;
    FmaCore<EV> core;
    int* vis = reinterpret_cast<int*>(core.carve(smem_raw, E));  // [F]
    int* pre = vis + a.F;                                        // [F+1]
    float* const Qs = core.Qs;
    float* const Ks = core.Ks;
    float* const Vs = core.Vs;
    int* const lim_s = core.lim_s;

    const int tid = threadIdx.x;

    pdl_wait();
    pdl_trigger();
    build_tile_prefix(a, kFmaTile, vis, pre);
    const int TH = pre[a.F];
    const int units = a.row_blocks * a.Hkv;
    const int64_t N = (int64_t)units * TH;
    const int ctas = effective_ctas(N, gridDim.x);
    if (blockIdx.x == 0 && tid == 0) {
        a.header[0] = TH;
        a.header[1] = ctas;
    }
    if (a.rq != nullptr && a.cos != nullptr)
        write_rotated_queries<T>(a.q, a.rq, a.cos, a.sin, a.F, a.W, a.Hq, a.S, a.E, a.R, blockIdx.x * kFmaThreads + tid,
                                 gridDim.x * kFmaThreads);
    if ((int)blockIdx.x >= ctas) return;

    const int64_t t0 = cta_first_tile(blockIdx.x, N, ctas), t1 = cta_first_tile(blockIdx.x + 1, N, ctas);
    const T* __restrict__ q = static_cast<const T*>(a.q);

    core.reset();

    int64_t u = t0 / TH;
    int j = (int)(t0 - u * TH);
    int cur_u = -1, cur_f = -1, fscan = 0, rb = 0, hkv = 0;
    for (int64_t t = t0; t < t1; ++t) {
        if ((int)u != cur_u) {
            cur_u = (int)u;
            cur_f = -1;
            fscan = 0;
            rb = cur_u / a.Hkv;
            hkv = cur_u % a.Hkv;
            core.reset();
        }
        while (j >= pre[fscan + 1]) ++fscan;
        const int f = fscan;
        if (f != cur_f) {
            cur_f = f;
            // (re)build the 16 query rows for this fragment: rotate, round to the storage type
#pragma unroll 4
            for (int idx = tid; idx < kFmaRows * E; idx += kFmaThreads) {
                const int r = idx / E, e = idx - r * E;
                const int gr = rb * kFmaRows + r;
                float val = 0.f;
                if (gr < a.rows_total) {
                    const RowId id = decode_row(gr, a.G, a.S);
                    const int hq = hkv * a.G + id.g;
                    if (a.cos != nullptr) {
                        const T* qrow = q + ((size_t)(id.w * a.Hq + hq) * a.S + id.s) * E;
                        const size_t tab = ((size_t)(f * a.W + id.w) * a.S + id.s) * a.R;
                        val = Scalar<T>::to_float(
                            Scalar<T>::from_float(rope_channel<T>(qrow, a.cos + tab, a.sin + tab, e, a.R)));
                    } else {
                        val = Scalar<T>::to_float(q[((size_t)((f * a.W + id.w) * a.Hq + hq) * a.S + id.s) * E + e]);
                    }
                }
                Qs[idx] = val;
            }
            if (tid < kFmaRows) {
                const int gr = rb * kFmaRows + tid;
                int lim = 0;
                if (gr < a.rows_total) {
                    const RowId id = decode_row(gr, a.G, a.S);
                    const int loc = a.loc[(f * a.W + id.w) * a.S + id.s];
                    lim = min(loc, vis[f] - 1) + 1;
                }
                lim_s[tid] = lim;
            }
        }
        const int tok0 = (j - pre[f]) * kFmaTile;
        const int ntok = min(kFmaTile, vis[f] - tok0);

        // ---- stage the K and V rows of this tile as fp32 (rows are consecutive in memory) ----
        {
            const size_t row0 = (size_t)hkv * a.ft.e[f].rows + tok0;
            const T* ksrc = static_cast<const T*>(a.ft.e[f].k) + row0 * E;
            const T* vsrc = static_cast<const T*>(a.ft.e[f].v) + row0 * EV;
            const int kvecs = ntok * E / VEC;
            for (int i = tid; i < kvecs; i += kFmaThreads) {
                const int4 raw = __ldg(reinterpret_cast<const int4*>(ksrc) + i);
                const T* x = reinterpret_cast<const T*>(&raw);
                const int idx = i * VEC, tok = idx / E, e = idx - tok * E;
#pragma unroll
                for (int k = 0; k < VEC; ++k) Ks[tok * (E + 1) + e + k] = Scalar<T>::to_float(x[k]);
            }
            const int vvecs = kFmaTile * EV / VEC, vvalid = ntok * EV / VEC;
            for (int i = tid; i < vvecs; i += kFmaThreads) {
                int4 raw = make_int4(0, 0, 0, 0);          // rows past the tile end must be finite
                if (i < vvalid) raw = __ldg(reinterpret_cast<const int4*>(vsrc) + i);
                const T* x = reinterpret_cast<const T*>(&raw);
#pragma unroll
                for (int k = 0; k < VEC; ++k) Vs[i * VEC + k] = Scalar<T>::to_float(x[k]);
            }
        }
        __syncthreads();

        core.compute(tok0, ntok, a.l2scale);

        // ---- leave a partial result where this CTA's share of the unit ends ----
        if (j == TH - 1 || t == t1 - 1) {
            int first, count;
            unit_ctas(u, TH, N, ctas, &first, &count);
            core.flush(a.ws_o, a.ws_m, a.ws_l, (size_t)u * a.parts_per_unit + (blockIdx.x - first));
        }
        __syncthreads();   // K/V/P/Q buffers are rewritten by the next tile
        if (++j == TH) {
            j = 0;
            ++u;
        }
    }
}

}  // namespace hogatt
