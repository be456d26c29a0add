// The steps either side of the attention op in a decode step:
//   * step_plan_kernel  -- per-step metadata: for every (fragment, worker, new token) the position of the
//     token relative to the start of that fragment in the worker's own ordering of the fragments, and the
//     cos/sin rows for it.  Restates the layer-0 block of HogwildCache.update
//     (python/hogwild/attention.py:164-204), which builds the same tensors with Python loops,
//     torch.stack and the model's rotary_emb on every step.
//   * append_kernel     -- K-side write path: rotate the new keys at their own positions and append keys
//     and values to the worker's fragment, in place, in preallocated [Hkv, capacity, E] slabs.  Restates
//     AttentionModule.forward's apply_rotary_pos_emb(key_states, cos, sin) followed by
//     HogwildCache.update's write_to[w].update(...) (python/hogwild/attention.py:315, :148-158), which
//     grows the fragment with torch.cat, and -- with one broadcast table row -- the re-rotation of
//     merge_caches (python/hogwild/attention.py:251-257).
#pragma once
#include "hogatt_device.cuh"

namespace hogatt {

constexpr int kMaxAppendSources = 64;

struct StepPlanArgs {
    int F, W, S, R;
    const int* order;          // [W][F] fragment ids in worker order, -1 after the last
    const int* lengths;        // [F] lengths including the S tokens being added
    const float* inv_freq;     // [R/2]
    float attention_scaling;
    int round_to;              // HOGATT_F32: keep fp32; HOGATT_F16 / HOGATT_BF16: round the table values through that type
    int* loc;                  // [F][W][S]
    float* cos;                // [F][W][S][R]
    float* sin;
};

// One CTA per (fragment, worker).  Thread 0 walks the worker's order backwards (at most F steps) to find
// the fragment's end position; all threads then fill the S x R table rows.
__global__ void __launch_bounds__(128) step_plan_kernel(const StepPlanArgs a) {
    const int f = blockIdx.x / a.W, w = blockIdx.x % a.W;
    __shared__ int s_end;
    if (threadIdx.x == 0) {
        // positions count from the end of the worker's sequence: the fragment that comes last in the order
        // ends at its own length, the one before it at the sum of both, ...  (attention.py:173-181)
        int n = 0;
        while (n < a.F && a.order[w * a.F + n] >= 0) ++n;
        int pos = 0, end = -1;
        for (int k = n - 1; k >= 0; --k) {
            const int g = a.order[w * a.F + k];
            pos += a.lengths[g];
            if (g == f) {
                end = pos;
                break;
            }
        }
        s_end = end;
    }
    __syncthreads();
    const int end = s_end;            // -1: this worker does not have the fragment at all
    const int half = a.R >> 1;
    for (int s = threadIdx.x; s < a.S; s += blockDim.x)
        a.loc[(f * a.W + w) * a.S + s] = end < 0 ? -1 : end - a.S + s;
    for (int i = threadIdx.x; i < a.S * half; i += blockDim.x) {
        const int s = i / half, c = i % half;
        const int p = end < 0 ? -1 : end - a.S + s;
        // fp32 product of the position and the inverse frequency, like rotary_emb's matmul of the two
        const float angle = __fmul_rn((float)p, a.inv_freq[c]);
        float sn, cs;
        sincosf(angle, &sn, &cs);
        cs = __fmul_rn(cs, a.attention_scaling);
        sn = __fmul_rn(sn, a.attention_scaling);
        if (a.round_to == HOGATT_F16) {
            cs = __half2float(__float2half_rn(cs));
            sn = __half2float(__float2half_rn(sn));
        } else if (a.round_to == HOGATT_BF16) {
            cs = __bfloat162float(__float2bfloat16_rn(cs));
            sn = __bfloat162float(__float2bfloat16_rn(sn));
        }
        const size_t row = ((size_t)(f * a.W + w) * a.S + s) * a.R;
        a.cos[row + c] = cs;
        a.cos[row + c + half] = cs;
        a.sin[row + c] = sn;
        a.sin[row + c + half] = sn;
    }
}

struct AppendArgs {
    int W, Hkv, E, Ev, S, R, F;
    int tables_lowp;                   // 0: fp32 tables, one rounding; 1: tables in the tensors' type, torch's three roundings
    int take_leading;                  // new_rows counts from the start of a source instead of from its end
    const void* k;
    const void* v;
    long long ks[3], vs[3];            // element strides of (source, kv head, row)
    const void* cos;
    const void* sin;
    long long ts[2];                   // element strides of (source, row); 0 broadcasts
    const int* new_rows;               // [W] or nullptr: only the last new_rows[w] rows of source w are appended
    int write_to[kMaxAppendSources];   // destination fragment per source
    const int* len_in;                 // [F]
    int* len_out;                      // [F], a different buffer
    int* status;
    FragmentTable ft;                  // destination slabs: k, v, rows = capacity
};

constexpr int STATUS_FRAGMENT_FULL = 256;      // an append did not fit into the fragment's slab; the overflow was dropped

// One rotated key channel in the tensors' own type, rounded the way torch rounds
// (x * cos) + (rotate_half(x) * sin) when all three tensors have that type: each product, then the sum.
template <class T>
__device__ __forceinline__ T rope_channel_lowp(const T* __restrict__ x, const T* __restrict__ c, const T* __restrict__ s,
                                               int e, int R) {
    const int half = R >> 1;
    if (e >= R) return x[e];
    const bool lo = e < half;
    const float xv = Scalar<T>::to_float(x[e]);
    const float yv = Scalar<T>::to_float(x[lo ? e + half : e - half]);
    const float a = Scalar<T>::to_float(Scalar<T>::from_float(__fmul_rn(xv, Scalar<T>::to_float(c[e]))));
    const float b = Scalar<T>::to_float(Scalar<T>::from_float(__fmul_rn(lo ? -yv : yv, Scalar<T>::to_float(s[e]))));
    return Scalar<T>::from_float(__fadd_rn(a, b));
}

// grid: (row chunks, kv heads, sources); a thread handles one 16-byte piece of a key row and of a value row
// when everything is 16-byte aligned, single elements otherwise.
template <class T>
__global__ void __launch_bounds__(256) append_kernel(const __grid_constant__ AppendArgs a, const int vectorised) {
    const int w = blockIdx.z, h = blockIdx.y;
    const int f = a.write_to[w];
    const int n = a.new_rows ? min(max(a.new_rows[w], 0), a.S) : a.S;
    const int skip = a.take_leading ? 0 : a.S - n;      // left-masked: the first rows of the source are padding
    int start = a.len_in[f];
    for (int w2 = 0; w2 < w; ++w2)                      // sources that share a fragment append in source order
        if (a.write_to[w2] == f) start += a.new_rows ? min(max(a.new_rows[w2], 0), a.S) : a.S;
    const int cap = a.ft.e[f].rows;
    const int fit = max(0, min(n, cap - start));
    if (fit < n && threadIdx.x == 0 && blockIdx.x == 0 && h == 0 && a.status) atomicOr(a.status, STATUS_FRAGMENT_FULL);

    // lengths: one thread of the whole grid, from len_in (nobody writes it)
    if (blockIdx.x == 0 && h == 0 && w == 0 && threadIdx.x < 32) {
        for (int g = threadIdx.x; g < a.F; g += 32) {
            int len = a.len_in[g];
            for (int w2 = 0; w2 < a.W; ++w2)
                if (a.write_to[w2] == g) len += a.new_rows ? min(max(a.new_rows[w2], 0), a.S) : a.S;
            a.len_out[g] = min(len, a.ft.e[g].rows);
        }
    }

    const T* ksrc = static_cast<const T*>(a.k) + w * a.ks[0] + h * a.ks[1];
    const T* vsrc = static_cast<const T*>(a.v) + w * a.vs[0] + h * a.vs[1];
    T* kdst = static_cast<T*>(const_cast<void*>(a.ft.e[f].k)) + ((size_t)h * cap + start) * a.E;
    T* vdst = static_cast<T*>(const_cast<void*>(a.ft.e[f].v)) + ((size_t)h * cap + start) * a.Ev;
    constexpr int VEC = 16 / (int)sizeof(T);
    const int kc = vectorised ? a.E / VEC : a.E, vc = vectorised ? a.Ev / VEC : a.Ev;     // pieces per row
    const int per_row = kc + vc;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < (int64_t)fit * per_row;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int r = (int)(i / per_row), c = (int)(i % per_row);
        const int sr = skip + r;
        if (c >= kc) {                                  // value piece: plain copy
            const int cv = c - kc;
            if (vectorised)
                *reinterpret_cast<uint4*>(vdst + (size_t)r * a.Ev + cv * VEC) =
                    *reinterpret_cast<const uint4*>(vsrc + sr * a.vs[2] + cv * VEC);
            else
                vdst[(size_t)r * a.Ev + cv] = vsrc[sr * a.vs[2] + cv];
            continue;
        }
        const T* krow = ksrc + sr * a.ks[2];
        const size_t tab = (size_t)(w * a.ts[0] + sr * a.ts[1]);
        if (!vectorised) {
            T out;
            if (a.tables_lowp || sizeof(T) == 4) {
                // same type everywhere; in fp32 this is also exactly the fp32-table arithmetic
                out = rope_channel_lowp<T>(krow, static_cast<const T*>(a.cos) + tab, static_cast<const T*>(a.sin) + tab, c, a.R);
            } else {
                out = Scalar<T>::from_float(rope_channel<T>(krow, static_cast<const float*>(a.cos) + tab,
                                                            static_cast<const float*>(a.sin) + tab, c, a.R));
            }
            kdst[(size_t)r * a.E + c] = out;
            continue;
        }
        if constexpr (sizeof(T) == 2) {
            uint4 out;
            if (a.tables_lowp) {
                T tmp[VEC];
#pragma unroll
                for (int e = 0; e < VEC; ++e)
                    tmp[e] = rope_channel_lowp<T>(krow, static_cast<const T*>(a.cos) + tab, static_cast<const T*>(a.sin) + tab,
                                                  c * VEC + e, a.R);
                out = *reinterpret_cast<const uint4*>(tmp);
            } else {
                out = rotate_chunk<T>(krow, static_cast<const float*>(a.cos) + tab, static_cast<const float*>(a.sin) + tab, c, a.R);
            }
            *reinterpret_cast<uint4*>(kdst + (size_t)r * a.E + c * VEC) = out;
        }
    }
}

}  // namespace hogatt
