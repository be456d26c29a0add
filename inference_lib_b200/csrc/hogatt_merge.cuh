// Split-K merge and the stand-alone query RoPE kernel.
#pragma once
#include "hogatt_device.cuh"

namespace hogatt {

constexpr int kMergeWarps = 4;

// One warp per output row: combine the partial results the attention CTAs left for the row's
// unit, normalise, round to the storage type.
//   out = sum_p O_p * 2^(m_p - M) / sum_p l_p * 2^(m_p - M),   M = max_p m_p
// Rows no key was visible to (every m_p = -inf, or no partial at all) come out as zeros.
// Same role as hogwild_attention_reduce_kernel (src/kernels/kernel_v21.cuh:605-656); that one
// folds normalised partials pairwise by their log-sum-exp, here the partials are unnormalised.
template <class T>
__global__ void __launch_bounds__(kMergeWarps * 32) merge_kernel(const __grid_constant__ KernelArgs a) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int u = blockIdx.x;
    const int rb = u / a.Hkv, hkv = u % a.Hkv;
    const int TH = a.header[0], ctas = a.header[1];
    const int units = a.row_blocks * a.Hkv;
    int first = 0, count = 0;
    if (TH > 0) unit_ctas(u, TH, (int64_t)units * TH, ctas, &first, &count);
    const int RPB = a.rows_per_block, Ev = a.Ev;
    T* __restrict__ out = static_cast<T*>(a.out);

    for (int row = blockIdx.y * kMergeWarps + warp; row < RPB; row += gridDim.y * kMergeWarps) {
        const int gr = rb * RPB + row;
        if (gr >= a.rows_total) continue;
        const RowId id = decode_row(gr, a.G, a.S);
        T* dst = out + ((size_t)(id.w * a.Hq + hkv * a.G + id.g) * a.S + id.s) * Ev;
        const size_t slot0 = (size_t)u * a.parts_per_unit;

        float M = -INFINITY;
        for (int p = lane; p < count; p += 32) M = fmaxf(M, a.ws_m[(slot0 + p) * RPB + row]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));

        float den = 0.f;
        if (M != -INFINITY) {
            for (int p = lane; p < count; p += 32)
                den += a.ws_l[(slot0 + p) * RPB + row] * exp2f(a.ws_m[(slot0 + p) * RPB + row] - M);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) den += __shfl_xor_sync(0xffffffffu, den, o);
        }
        const bool blind = !(den > 0.f);
        const float inv = blind ? 0.f : 1.f / den;

        for (int e = lane * 4; e < Ev; e += 128) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            if (!blind) {
                for (int p = 0; p < count; ++p) {
                    const float wgt = exp2f(a.ws_m[(slot0 + p) * RPB + row] - M);
                    const float4 x = *reinterpret_cast<const float4*>(a.ws_o + ((slot0 + p) * RPB + row) * Ev + e);
                    acc.x = fmaf(x.x, wgt, acc.x);
                    acc.y = fmaf(x.y, wgt, acc.y);
                    acc.z = fmaf(x.z, wgt, acc.z);
                    acc.w = fmaf(x.w, wgt, acc.w);
                }
            }
            dst[e + 0] = Scalar<T>::from_float(acc.x * inv);
            dst[e + 1] = Scalar<T>::from_float(acc.y * inv);
            dst[e + 2] = Scalar<T>::from_float(acc.z * inv);
            dst[e + 3] = Scalar<T>::from_float(acc.w * inv);
        }
    }
}

// rq[f,w,h,s,:] = rope(q[w,h,s,:], cos[f,w,s,:], sin[f,w,s,:]); one warp per output row.
// Replaces rope_kernel (src/rope.cuh:2-52), which uses one thread per channel and one CTA per row.
template <class T>
__global__ void __launch_bounds__(128) rope_kernel(T* __restrict__ rq, const T* __restrict__ q,
                                                   const float* __restrict__ cosines,
                                                   const float* __restrict__ sines, int F, int W, int Hq, int S,
                                                   int E, int R) {
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (row >= F * W * Hq * S) return;
    int s = row % S;
    int t = row / S;
    const int h = t % Hq;
    t /= Hq;
    const int w = t % W;
    const int f = t / W;
    const T* qrow = q + ((size_t)(w * Hq + h) * S + s) * E;
    const float* c = cosines + ((size_t)(f * W + w) * S + s) * R;
    const float* sn = sines + ((size_t)(f * W + w) * S + s) * R;
    T* dst = rq + (size_t)row * E;
    for (int e = lane; e < E; e += 32) dst[e] = Scalar<T>::from_float(rope_channel<T>(qrow, c, sn, e, R));
}

}  // namespace hogatt
