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
struct FragmentEntry {                     // 24 bytes: one constant-cache line holds a fragment's whole entry
    const void* k;                         // [Hkv, rows, E]
    const void* v;                         // [Hkv, rows, Ev]
    int rows;                              // token extent of the tensors (head stride = rows * E)
    int vis;                               // host plan: upper bound of the visible rows, 0 <= vis <= rows
};
struct FragmentTable {
    FragmentEntry e[HOGATT_MAX_FRAGMENTS];
};

struct KernelArgs {
    int F, W, Hq, Hkv, G, E, Ev, S, R;
    int rows_total;        // W * G * S query rows per kv head
    int rows_per_block;    // rows one CTA keeps resident (16 * m-tiles)
    int row_blocks;        // ceil(rows_total / rows_per_block)
    int parts_per_unit;    // partial-result slots reserved per unit in the workspace
    // Host plan (tensor-core kernel, persistent grid): the tiles come from ft.e[f].vis alone, nothing is read
    // from device memory to build them; plan_tiles = tiles per unit, plan_ctas = CTAs that get work.
    int host_plan, plan_tiles, plan_ctas;
    int stable_fragments;  // fragments [0, stable_fragments) may be fetched before griddepcontrol.wait
    int debug_id;          // tuning builds only: which slot of the event trace this call writes (0 otherwise)
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
    // Fused output all-gather over peer memory (KV-head sharding): when world > 0 the merge step stores
    // every finished output row into the full-size output of EVERY rank (plain stores through peer
    // pointers) at this rank's head offset, instead of into `out`.
    int world, rank;       // world == 0: no gather
    void* peer_out[HOGATT_MAX_PEERS];      // [W, world * Hq, S, Ev] on each rank, mapped into this GPU's address space
    FragmentTable ft;
};

enum DeviceStatusBits : int {
    STATUS_WAIT_FULL_TIMEOUT = 1,     // a consumer gave up waiting for a KV tile
    STATUS_WAIT_EMPTY_TIMEOUT = 2,    // the producer gave up waiting for a free stage
    STATUS_WAIT_SYNC_TIMEOUT = 4,     // consumer warps gave up waiting for each other
    STATUS_DRAIN_TIMEOUT = 8,         // copies still in flight when the CTA wanted to leave
    STATUS_WAIT_PEER_TIMEOUT = 32     // a peer GPU never reported its share of a gathered output
};

// Optional timeline for kernel tuning (compile with -DHOGATT_TIMELINE=<cta>): lane 0 of two warps of
// one CTA records clock64() at named points into a device array that a debug entry point copies out.
#ifdef HOGATT_TIMELINE
__device__ long long g_timeline[2][1024];
__device__ int g_timeline_tag[2][1024];
__device__ int g_timeline_n[2];
__device__ unsigned long long g_cta_t[3][256];   // per CTA: start, first tile consumed, end (globaltimer ns)
__device__ unsigned int g_cta_sm[256];
__device__ unsigned long long g_span[8];      // [0] attn first start, [1] attn last end, [2] merge first start, [3] merge last end
// Per call (kernel argument debug_id, a counter the host keeps in these builds) and per CTA: globaltimer stamps of
// named events of the attention kernel, and first start / last end of the merge kernel.
constexpr int kTraceCalls = 64, kTraceEvents = 8;
__device__ unsigned long long g_trace[kTraceCalls][kTraceEvents][256];
__device__ unsigned long long g_mtrace[kTraceCalls][2];
__device__ unsigned long long g_strace[kTraceCalls][4];
__device__ unsigned long long g_mphase[kTraceCalls][4][128];  // merge CTAs: start, wait over, first row combined, end     // exchange kernel: start, predecessor done, published, peers seen
#define HOGATT_TRACE(id, ev) do { if (blockIdx.x < 256) g_trace[(id) % kTraceCalls][ev][blockIdx.x] = global_timer_ns_(); } while (0)
#define HOGATT_SPAN_MIN(i) do { if (threadIdx.x == 0) atomicMin(&g_span[i], global_timer_ns_()); } while (0)
#define HOGATT_SPAN_MAX(i) do { if (threadIdx.x == 0) atomicMax(&g_span[i], global_timer_ns_()); } while (0)
__device__ __forceinline__ unsigned long long global_timer_ns_() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define HOGATT_TL_DECL int tlc__ = 0
#define HOGATT_TL(who, tag)                                                              \
    do {                                                                                 \
        if (blockIdx.x == HOGATT_TIMELINE && (threadIdx.x & 31) == 0 && tlc__ < 1024) {  \
            g_timeline[who][tlc__] = clock64();                                          \
            g_timeline_tag[who][tlc__] = (tag);                                          \
            g_timeline_n[who] = ++tlc__;                                                 \
        }                                                                                \
    } while (0)
#else
#define HOGATT_TL_DECL
#define HOGATT_TL(who, tag)
#define HOGATT_TRACE(id, ev)
#define HOGATT_SPAN_MIN(i)
#define HOGATT_SPAN_MAX(i)
#endif

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
// `q` points at the un-rotated row, `c`/`s` at that row's table for the fragment.  Written without
// branches (selects only) so that the loads of many channels can be issued back to back instead of
// one dependent round trip per channel.
template <class T>
__device__ __forceinline__ float rope_channel(const T* __restrict__ q, const float* __restrict__ c,
                                              const float* __restrict__ s, int e, int R) {
    const int half = R >> 1;
    const bool rot = e < R, lo = e < half;
    const int pe = rot ? (lo ? e + half : e - half) : e;    // partner channel
    const int te = rot ? e : 0;                              // table index (always in range)
    const float x = Scalar<T>::to_float(q[e]);
    const float y = Scalar<T>::to_float(q[pe]);
    const float a = __fmul_rn(x, c[te]), b = __fmul_rn(y, s[te]);
    const float r = lo ? __fsub_rn(a, b) : __fadd_rn(a, b);
    return rot ? r : x;
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
// The limit the kernels read (only on the slow path of a wait): one second unless the host was started with
// HOGATT_WAIT_LIMIT_MS in the environment, which the library copies here once per device (tests of the give-up path).
__device__ unsigned long long g_wait_limit_ns = kWaitLimitNs;

// The polling loop lives out of line: these kernels run for microseconds and their instruction fetch
// shows in the call time, so every wait site is just a try_wait and a call.
__device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int bit);
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                                  int* status, int bit) {
    if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_slow(bar, parity, abort_flag, status, bit);
}
__device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int bit) {
    const uint64_t t0 = global_timer_ns();
    uint32_t spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++spins & 63u) == 0) {
            if (*abort_flag) return false;
            if (global_timer_ns() - t0 > g_wait_limit_ns) {
                *abort_flag = 1;
                if (status) atomicOr(status, bit);
                return false;
            }
        }
    }
    return true;
}

// Programmatic dependent launch: a kernel launched with the "programmatic stream serialization"
// attribute may start while its predecessor in the stream is still running; it must call
// pdl_wait() before it touches anything the predecessor reads or writes.  pdl_trigger() lets the
// NEXT kernel in the stream start being scheduled.  Both are no-ops for a normal launch.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- thread-block cluster helpers (distributed shared memory) -----------------------------------------
// barrier.cluster is a hardware barrier over every thread of every CTA of the cluster (like bar.sync over
// a CTA): it cannot be polled, so every thread of a cluster kernel must reach each of them exactly once,
// whatever else went wrong before (all other waits in these kernels are bounded).
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_nctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
}
// Address of the same shared-memory location in CTA `rank` of this cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ float4 ld_cluster_f4(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "r"(addr)
                 : "memory");
    return v;
}
__device__ __forceinline__ float ld_cluster_f(uint32_t addr) {
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
    return v;
}
// bar.sync over `threads` threads (a multiple of 32) on hardware barrier `id` (1..15; 0 is __syncthreads).
__device__ __forceinline__ void named_barrier_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
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

// Two adjacent rotated channels (e even) of a 16-bit query row, packed for an MMA A-fragment.
// Needs R % 4 == 0 so that e and e + 1 lie on the same side of R/2 and of R; 4- and 8-byte loads.
template <class T>
__device__ __forceinline__ uint32_t rope_pair(const T* __restrict__ q, const float* __restrict__ c,
                                              const float* __restrict__ s, int e, int R) {
    const int half = R >> 1;
    const bool rot = e < R, lo = e < half;
    const int pe = rot ? (lo ? e + half : e - half) : e;
    const int te = rot ? e : 0;
    const uint32_t xr = *reinterpret_cast<const uint32_t*>(q + e);
    const uint32_t yr = *reinterpret_cast<const uint32_t*>(q + pe);
    const float2 cv = *reinterpret_cast<const float2*>(c + te);
    const float2 sv = *reinterpret_cast<const float2*>(s + te);
    const T* xp = reinterpret_cast<const T*>(&xr);
    const T* yp = reinterpret_cast<const T*>(&yr);
    const float x0 = Scalar<T>::to_float(xp[0]), x1 = Scalar<T>::to_float(xp[1]);
    const float y0 = Scalar<T>::to_float(yp[0]), y1 = Scalar<T>::to_float(yp[1]);
    const float a0 = __fmul_rn(x0, cv.x), b0 = __fmul_rn(y0, sv.x);
    const float a1 = __fmul_rn(x1, cv.y), b1 = __fmul_rn(y1, sv.y);
    const float r0 = lo ? __fsub_rn(a0, b0) : __fadd_rn(a0, b0);
    const float r1 = lo ? __fsub_rn(a1, b1) : __fadd_rn(a1, b1);
    return rot ? pack2<T>(r0, r1) : xr;
}

// Eight adjacent rotated channels [8*ch, 8*ch + 8) of a 16-bit query row as one 16-byte vector.
// All loads are 16-byte vectors and independent of each other, so a thread can keep several chunks
// in flight in a single memory round trip.  Needs R % 16 == 0 (the partner of a chunk is a whole
// chunk) and 16-byte aligned table rows.
template <class T>
__device__ __forceinline__ uint4 rotate_chunk(const T* __restrict__ q, const float* __restrict__ c,
                                              const float* __restrict__ s, int ch, int R) {
    const int e0 = ch * 8, half = R >> 1;
    const bool rot = e0 < R, lo = e0 < half;
    const int pe = rot ? (lo ? e0 + half : e0 - half) : e0;
    const int te = rot ? e0 : 0;
    const uint4 xr = *reinterpret_cast<const uint4*>(q + e0);
    const uint4 yr = *reinterpret_cast<const uint4*>(q + pe);
    const float4 c0 = *reinterpret_cast<const float4*>(c + te), c1 = *reinterpret_cast<const float4*>(c + te + 4);
    const float4 s0 = *reinterpret_cast<const float4*>(s + te), s1 = *reinterpret_cast<const float4*>(s + te + 4);
    const T* x = reinterpret_cast<const T*>(&xr);
    const T* y = reinterpret_cast<const T*>(&yr);
    const float cv[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float sv[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    uint4 out;
    uint32_t* o = reinterpret_cast<uint32_t*>(&out);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float r[2];
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const float a = __fmul_rn(Scalar<T>::to_float(x[2 * i + k]), cv[2 * i + k]);
            const float b = __fmul_rn(Scalar<T>::to_float(y[2 * i + k]), sv[2 * i + k]);
            r[k] = lo ? __fsub_rn(a, b) : __fadd_rn(a, b);
        }
        o[i] = pack2<T>(r[0], r[1]);
    }
    return rot ? out : xr;
}

// True when rotate_chunk can be used for this call.
__device__ __forceinline__ bool chunked_rope_ok(const float* c, const float* s, int R, int E) {
    return (R & 15) == 0 && (E & 7) == 0 && ((((uintptr_t)c) | ((uintptr_t)s)) & 15u) == 0;
}

// rq[f,w,h,s,:] for all rows, dealt over the participating threads of the whole grid
// (`gthread` of `gthreads`).  Used when the caller wants the rotated queries back.  16-bit types
// take the chunked path: one 16-byte chunk per thread per step, one memory round trip.
template <class T>
__device__ __noinline__ void write_rotated_queries(const void* qv, void* rqv, const float* __restrict__ cos,
                                                   const float* __restrict__ sin, int F, int W, int Hq, int S, int E, int R,
                                                   int gthread, int gthreads) {
    T* __restrict__ rq = static_cast<T*>(rqv);
    const T* __restrict__ q = static_cast<const T*>(qv);
    const int rows = F * W * Hq * S;
    if constexpr (sizeof(T) == 2) {
      if (chunked_rope_ok(cos, sin, R, E)) {
        const int cpr = E >> 3;
        const int items = rows * cpr;
        // four chunks per pass with all their loads in flight together (nothing here aliases): when one warp
        // writes the whole share of its CTA in the middle of the K/V stream, a load takes 1.5-2 us
#pragma unroll 4
        for (int item = gthread; item < items; item += gthreads) {
            const int row = item / cpr, ch = item - row * cpr;
            const int s = row % S;
            int t = row / S;
            const int h = t % Hq;
            t /= Hq;
            const int w = t % W, f = t / W;
            const T* qrow = q + ((size_t)(w * Hq + h) * S + s) * E;
            const size_t tab = ((size_t)(f * W + w) * S + s) * R;
            const uint4 val = rotate_chunk<T>(qrow, cos + tab, sin + tab, ch, R);
            *reinterpret_cast<uint4*>(rq + (size_t)row * E + ch * 8) = val;
        }
        return;
      }
    }
    const int64_t items = (int64_t)rows * E;
#pragma unroll 1
    for (int64_t item = gthread; item < items; item += gthreads) {
        const int row = (int)(item / E), e = (int)(item - (int64_t)row * E);
        const int s = row % S;
        int t = row / S;
        const int h = t % Hq;
        t /= Hq;
        const int w = t % W, f = t / W;
        const T* qrow = q + ((size_t)(w * Hq + h) * S + s) * E;
        const size_t tab = ((size_t)(f * W + w) * S + s) * R;
        rq[item] = Scalar<T>::from_float(rope_channel<T>(qrow, cos + tab, sin + tab, e, R));
    }
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
    // (loops kept rolled on purpose: this runs once per CTA and its instruction fetch is on the start-up path)
#pragma unroll 1
    for (int f = warp; f < a.F; f += nwarps) {
        int top = -1;
        int cap = a.ft.e[f].rows;
        if (a.flen) cap = min(cap, a.flen[f]);            // issued together with the loads below
#pragma unroll 1
        for (int i = lane; i < per; i += 32) top = max(top, a.loc[f * per + i]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) top = max(top, __shfl_xor_sync(0xffffffffu, top, o));
        if (lane == 0) vis[f] = max(0, min(top, cap - 1) + 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int acc = 0;
#pragma unroll 1
        for (int f = 0; f < a.F; ++f) {
            pre[f] = acc;
            acc += ceil_div(vis[f], tile_tokens);
        }
        pre[a.F] = acc;
    }
    __syncthreads();
}

// Host plan: the same two arrays from the kernel arguments alone -- vis[f] is the host's upper bound of the
// visible rows -- so that nothing is read from device memory before the first K/V copy can be issued.
// Called by ONE whole warp; the caller synchronises the CTA afterwards.
__device__ __forceinline__ void host_tile_prefix(const KernelArgs& a, int tile_tokens, int* vis, int* pre) {
    const int lane = threadIdx.x & 31;
    int carry = 0;
#pragma unroll 1
    for (int f0 = 0; f0 < a.F; f0 += 32) {
        const int f = f0 + lane;
        const int v = f < a.F ? a.ft.e[f].vis : 0;
        const int mine = ceil_div(v, tile_tokens);
        int x = mine;                                      // inclusive scan over the warp
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int y = __shfl_up_sync(0xffffffffu, x, o);
            if (lane >= o) x += y;
        }
        if (f < a.F) {
            vis[f] = v;
            pre[f] = carry + x - mine;
        }
        carry += __shfl_sync(0xffffffffu, x, 31);
    }
    if (lane == 0) pre[a.F] = carry;
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
