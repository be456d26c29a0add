// Device-side building blocks shared by the attention kernels: the by-value kernel arguments,
// sm_100a PTX wrappers (mbarrier, bulk async copy, ldmatrix, mma), bounded waits, the tile walker.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/hogatt.h"
#include "hogatt_plan.h"

namespace hogatt {

// ---------------------------------------------------------------------------------------------
// Kernel arguments.  Everything travels by value (`__grid_constant__`), including the fragment
// table, so a call needs no host->device copy of pointers (the reference copies a pointer table
// per call, src/binding.cu:79-103).
// ---------------------------------------------------------------------------------------------
struct FragmentTable {
    const void* k[HOGATT_MAX_FRAGMENTS];   // [Hkv, rows, E]
    const void* v[HOGATT_MAX_FRAGMENTS];   // [Hkv, rows, Ev]
    int rows[HOGATT_MAX_FRAGMENTS];        // token extent of the tensors (head stride = rows * E)
};

struct KernelArgs {
    int F, W, Hq, Hkv, G, E, Ev, S, R;
    int rows_total;        // W * G * S query rows per kv head
    int rows_per_block;    // rows one CTA keeps resident (16 * m-tiles)
    int row_blocks;        // ceil(rows_total / rows_per_block)
    int parts_per_unit;    // partial-result slots reserved per unit in the workspace
    float l2scale;         // scale * log2(e): softmax runs in base 2
    void* out;
    void* rq;              // optional rotated-query output
    const void* q;         // [W,Hq,S,E] if cos != nullptr else [F,W,Hq,S,E]
    const float* cos;
    const float* sin;
    const int* loc;
    const int* flen;       // optional device lengths
    int* header;           // workspace: {tiles per unit, CTAs with work}
    float* ws_o;           // [units][parts][rows_per_block][Ev]
    float* ws_m;           // [units][parts][rows_per_block]   running max (base-2, scaled)
    float* ws_l;           // [units][parts][rows_per_block]   running sum
    int* status;           // optional
    FragmentTable ft;
};

enum DeviceStatusBits : int {
    STATUS_WAIT_FULL_TIMEOUT = 1,     // a consumer gave up waiting for a KV tile
    STATUS_WAIT_EMPTY_TIMEOUT = 2,    // the producer gave up waiting for a free stage
    STATUS_WAIT_SYNC_TIMEOUT = 4,     // consumer warps gave up waiting for each other
    STATUS_DRAIN_TIMEOUT = 8          // copies still in flight when the CTA wanted to leave
};

// ---------------------------------------------------------------------------------------------
// Scalar type helpers
// ---------------------------------------------------------------------------------------------
template <class T> struct Scalar;
template <> struct Scalar<float> {
    static __device__ __forceinline__ float to_float(float x) { return x; }
    static __device__ __forceinline__ float from_float(float x) { return x; }
};
template <> struct Scalar<__half> {
    static __device__ __forceinline__ float to_float(__half x) { return __half2float(x); }
    static __device__ __forceinline__ __half from_float(float x) { return __float2half_rn(x); }
};
template <> struct Scalar<__nv_bfloat16> {
    static __device__ __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }
    static __device__ __forceinline__ __nv_bfloat16 from_float(float x) { return __float2bfloat16_rn(x); }
};

// One rotated query channel, computed exactly like the reference's eager path: both products are
// rounded to fp32 before they are added (no fused multiply-add), and the caller rounds the sum
// to the storage type (python/hogwild/attention.py:84-90; src/rope.cuh:24-46, src/q_rope.h:17-25).
// `q` points at the un-rotated row, `c`/`s` at that row's table for the fragment.
template <class T>
__device__ __forceinline__ float rope_channel(const T* __restrict__ q, const float* __restrict__ c,
                                              const float* __restrict__ s, int e, int R) {
    const float x = Scalar<T>::to_float(q[e]);
    if (e >= R) return x;
    const int half = R >> 1;
    if (e < half) {
        const float y = Scalar<T>::to_float(q[e + half]);
        return __fsub_rn(__fmul_rn(x, c[e]), __fmul_rn(y, s[e]));
    }
    const float y = Scalar<T>::to_float(q[e - half]);
    return __fadd_rn(__fmul_rn(x, c[e]), __fmul_rn(y, s[e]));
}

// ---------------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}" ::"r"(bar),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Every wait in these kernels is bounded: after about a second without progress the waiter
// records `bit` in the caller's status word, raises the CTA-wide abort flag and reports failure,
// and every loop that sees a failed wait or the flag leaves without touching the tile.
constexpr uint64_t kWaitLimitNs = 1000ull * 1000ull * 1000ull;

__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                                  int* status, int bit) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = global_timer_ns();
    uint32_t spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++spins & 63u) == 0) {
            if (*abort_flag) return false;
            if (global_timer_ns() - t0 > kWaitLimitNs) {
                *abort_flag = 1;
                if (status) atomicOr(status, bit);
                return false;
            }
        }
    }
    return true;
}

// generic-proxy writes -> later async-proxy (bulk copy) writes to the same shared memory
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// 1-D bulk async copy global -> this CTA's shared memory, completion counted in bytes on `bar`.
// Source, destination and size must be multiples of 16 bytes.
__device__ __forceinline__ void bulk_load(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     dst_smem),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void bulk_load_hint(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar,
                                               uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::
            "r"(dst_smem),
        "l"(src), "r"(bytes), "r"(bar), "l"(policy)
        : "memory");
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                                  uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}

template <class T>
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma_16816<__nv_bfloat16>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma_16816<__half>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <class T>
__device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// ---------------------------------------------------------------------------------------------
// Visible lengths and the tile prefix, built once per CTA in shared memory.
//   vis[f]  = clamp(max over (w,s) of loc[f,w,s] + 1, 0, min(rows_f, flen[f]))
//   pre[f]  = tiles of fragments 0..f-1;  pre[F] = tiles per unit
// Must be called by all threads of the CTA; ends with a __syncthreads().
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void build_tile_prefix(const KernelArgs& a, int tile_tokens, int* vis, int* pre) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int per = a.W * a.S;
    for (int f = warp; f < a.F; f += nwarps) {
        int top = -1;
        for (int i = lane; i < per; i += 32) top = max(top, a.loc[f * per + i]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) top = max(top, __shfl_xor_sync(0xffffffffu, top, o));
        if (lane == 0) {
            int cap = a.ft.rows[f];
            if (a.flen) cap = min(cap, a.flen[f]);
            vis[f] = max(0, min(top + 1, cap));
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int acc = 0;
        for (int f = 0; f < a.F; ++f) {
            pre[f] = acc;
            acc += ceil_div(vis[f], tile_tokens);
        }
        pre[a.F] = acc;
    }
    __syncthreads();
}

// Row bookkeeping: query row r of a kv head (0 <= r < W*G*S) is worker w, group head g, token s
// with s fastest, so the rows of one (worker, head) are adjacent.
struct RowId {
    int w, g, s;
};
__device__ __forceinline__ RowId decode_row(int r, int G, int S) {
    RowId id;
    id.s = r % S;
    const int t = r / S;
    id.g = t % G;
    id.w = t / G;
    return id;
}

}  // namespace hogatt
