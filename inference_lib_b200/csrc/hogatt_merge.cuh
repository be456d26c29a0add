// Split-K merge and the stand-alone query RoPE kernel.
#pragma once
#include "hogatt_device.cuh"

namespace hogatt {

constexpr int kMergeWarps = 4;

// Four consecutive output values as ONE store (8 bytes of 16-bit values, 16 bytes of fp32).  `dst` is aligned to
// that: outputs are 16-byte aligned, rows are Ev values long and a lane's first column is a multiple of four.  Over
// NVLink (the output rows of a sharded call go to every peer) four 2-byte stores per lane were four partial-sector
// writes per 8 bytes.
template <class T>
__device__ __forceinline__ void store4(T* dst, float a, float b, float c, float d) {
    if constexpr (sizeof(T) == 2) {
        *reinterpret_cast<uint2*>(dst) = make_uint2(pack2<T>(a, b), pack2<T>(c, d));
    } else {
        *reinterpret_cast<float4*>(dst) = make_float4(a, b, c, d);
    }
}

// Combine the partial results of one output row (one warp), normalise, round to the storage type.
//   out = sum_p O_p * 2^(m_p - M) / sum_p l_p * 2^(m_p - M),   M = max_p m_p
// A row no key was visible to (every m_p = -inf, or no partial at all) comes out as zeros.
// Partial p of the row lives at ws_o[(slot0 + p) * rpb + row][:], ws_m / ws_l likewise.
// Same role as hogwild_attention_reduce_kernel (src/kernels/kernel_v21.cuh:605-656); that one
// folds normalised partials pairwise by their log-sum-exp, here the partials are unnormalised.
// The statistics of all partials (lane-strided) and the lane's four output columns of the first kBatch
// partials are all loaded before any is used: one memory round trip at 8 kv heads per GPU (19-20 partials
// per row); every further batch of kBatch partials (fewer kv heads, more partials each) is one more.
// `slots` partial slots exist for the row (an argument of the launch); how many of them hold a partial
// (`count`) may itself come from memory: `count_of()` is evaluated only after the loads of the
// statistics and of the first batch have been issued for ALL slots, so that the count's own load shares
// their round trip; what an unused slot returned is discarded (selected away, never multiplied).
// One call handles 128 output columns (head sizes up to 128: the whole row); wider rows call it again.
template <class T, int kMaxStat, int kBatch, class CountFn>
__device__ __forceinline__ void merge_partials_rows(const float* __restrict__ ws_o, const float* __restrict__ ws_m,
                                                   const float* __restrict__ ws_l, size_t slot0, int rpb, int Ev,
                                                   int row, int slots, CountFn count_of, T* const* bases, int nbases,
                                                   size_t offset, int lane, int e0, unsigned long long* stamp = nullptr) {
    // kBatch: output partials fetched in the first round trip (24; 4 or 8 where a row never has more: a unit of
    // many query rows is cut into few partials, and a lean kernel keeps 16 CTAs per SM resident instead of 3).
    // kMaxStat: statistics held per lane (32 * kMaxStat partials per row without extra loads)
    const int pstride = rpb * Ev;                    // floats between consecutive partials of a row (32-bit offsets: less code)
    float mp[kMaxStat], lp[kMaxStat];
#pragma unroll
    for (int k = 0; k < kMaxStat; ++k) {
        const int p = lane + 32 * k;
        const bool have = p < slots;
        mp[k] = have ? __ldcg(ws_m + (slot0 + p) * rpb + row) : -INFINITY;
        lp[k] = have ? __ldcg(ws_l + (slot0 + p) * rpb + row) : 0.f;
    }
    int count = 0;
    float M = -INFINITY, inv = 0.f;
    bool blind = true;
    {                                               // columns e0 .. e0 + 127 of the row; every lane takes part (shuffles)
        const int e = e0 + lane * 4;
        const bool mine = e < Ev;
        const float* src = ws_o + (slot0 * rpb + row) * Ev + (mine ? e : 0);
        float4 x[kBatch];
        const int last_slot = slots - 1;             // slots past the last one re-read it (always a valid address)
#pragma unroll
        for (int k = 0; k < kBatch; ++k)
            x[k] = __ldcg(reinterpret_cast<const float4*>(src + min(k, last_slot) * pstride));
        {
            count = count_of();
#pragma unroll
            for (int k = 0; k < kMaxStat; ++k)
                if (lane + 32 * k >= count) {
                    mp[k] = -INFINITY;
                    lp[k] = 0.f;
                }
            // weights 2^(m_p - M) (kept in mp[]) and the denominator
            M = mp[0];
#pragma unroll
            for (int k = 1; k < kMaxStat; ++k) M = fmaxf(M, mp[k]);
            if (kMaxStat > 1)
                for (int p = lane + 32 * kMaxStat; p < count; p += 32) M = fmaxf(M, __ldcg(ws_m + (slot0 + p) * rpb + row));
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
            const bool dark = M == -INFINITY;
            float den = 0.f;
#pragma unroll
            for (int k = 0; k < kMaxStat; ++k) {
                mp[k] = dark ? 0.f : exp2f(mp[k] - M);
                den = fmaf(lp[k], mp[k], den);
            }
            if (kMaxStat > 1 && !dark)
                for (int p = lane + 32 * kMaxStat; p < count; p += 32)
                    den += __ldcg(ws_l + (slot0 + p) * rpb + row) * exp2f(__ldcg(ws_m + (slot0 + p) * rpb + row) - M);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) den += __shfl_xor_sync(0xffffffffu, den, o);
            blind = !(den > 0.f);
            inv = blind ? 0.f : 1.f / den;
#ifdef HOGATT_TIMELINE
            if (stamp && lane == 0) *stamp = global_timer_ns_();      // the statistics have arrived
#endif
        }
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int k = 0; k < kBatch; ++k) {          // kBatch <= 32: the weights of the first batch sit in mp[0]
            const float wgt = __shfl_sync(0xffffffffu, mp[0], k);
            const bool used = k < count;            // an unused slot may hold anything, NaN included: select, do not multiply
            acc.x = fmaf(used ? x[k].x : 0.f, wgt, acc.x);
            acc.y = fmaf(used ? x[k].y : 0.f, wgt, acc.y);
            acc.z = fmaf(used ? x[k].z : 0.f, wgt, acc.z);
            acc.w = fmaf(used ? x[k].w : 0.f, wgt, acc.w);
        }
        // more partials: one round trip per further batch.  The lean instantiation (at most 32 partials) only has
        // 8 left; it is kept small on purpose -- this kernel runs for 2.5 us and its instruction fetch shows.
        constexpr int kNext = (kMaxStat == 1 && kBatch > 16) ? (kBatch < 32 ? 32 - kBatch : 8) : kBatch;   // (never 0: the loop must advance)
#pragma unroll 1
        for (int p0 = kBatch; p0 < count; p0 += kNext) {
#pragma unroll
            for (int k = 0; k < kNext; ++k)
                x[k] = __ldcg(reinterpret_cast<const float4*>(src + min(p0 + k, count - 1) * pstride));
#pragma unroll
            for (int k = 0; k < kNext; ++k) {
                const int p = p0 + k;                           // warp-uniform
                float wsel = mp[0];
#pragma unroll
                for (int q = 1; q < kMaxStat; ++q) wsel = ((p >> 5) == q) ? mp[q] : wsel;
                float wgt = __shfl_sync(0xffffffffu, wsel, p & 31);
                if (kMaxStat > 1 && p >= 32 * kMaxStat)         // beyond the per-lane table
                    wgt = (blind || p >= count) ? 0.f : exp2f(__ldcg(ws_m + (slot0 + p) * rpb + row) - M);
                acc.x = fmaf(x[k].x, wgt, acc.x);
                acc.y = fmaf(x[k].y, wgt, acc.y);
                acc.z = fmaf(x[k].z, wgt, acc.z);
                acc.w = fmaf(x[k].w, wgt, acc.w);
            }
        }
        if (blind) acc = make_float4(0.f, 0.f, 0.f, 0.f);
        if (mine) {
            for (int b = 0; b < nbases; ++b)            // one destination, or the full-size output of every rank
                store4<T>(bases[b] + offset + e, acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
        }
    }
}

// Split-K merge of the fragment op: grid (units, row groups), one warp per output row.
// NSTAT = 1 serves up to 32 partials per row (8 kv heads on 148 SMs: 19-20), NSTAT = 5 up to 160 without
// extra loads (kv heads sharded over GPUs: 37, 74, 148 partials per row); the host picks by the number of
// partial slots per unit.  Two kernels rather than one with both paths: the bigger code cost the common
// case +1 us per call (instruction fetch of a kernel that runs for 2.5 us).
template <class T, int NSTAT, int KB = 24, int MW = kMergeWarps>
__global__ void __launch_bounds__(MW * 32) merge_kernel(const __grid_constant__ KernelArgs a) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int u = blockIdx.x;
    const int rb = u / a.Hkv, hkv = u % a.Hkv;
    HOGATT_SPAN_MIN(2);
#ifdef HOGATT_TIMELINE
    if (threadIdx.x == 0) atomicMin(&g_mtrace[a.debug_id % kTraceCalls][0], global_timer_ns_());
#endif
#ifdef HOGATT_TIMELINE
    const int mcta = blockIdx.y * gridDim.x + blockIdx.x;
    if (threadIdx.x == 0 && mcta < 128) g_mphase[a.debug_id % kTraceCalls][0][mcta] = global_timer_ns_();
#endif
    pdl_trigger();       // the next call's attention kernel may queue up behind this grid
    const int units = a.row_blocks * a.Hkv;
    const int RPB = a.rows_per_block, Ev = a.Ev;
    // how many CTAs left a partial for this unit: from the header the attention kernel wrote
    // (under a host plan both numbers are kernel arguments)
    const int* hdr = a.header;
    const int host_plan = a.host_plan, plan_tiles = a.plan_tiles, plan_ctas = a.plan_ctas;
    auto count_of = [=]() {
        const int TH = host_plan ? plan_tiles : __ldcg(hdr), ctas = host_plan ? plan_ctas : __ldcg(hdr + 1);
        int first = 0, count = 0;
        if (TH > 0) unit_ctas(u, TH, (int64_t)units * TH, ctas, &first, &count);
        return count;
    };
    T* const local_out = static_cast<T*>(a.out);
    T* const* bases = a.world > 0 ? reinterpret_cast<T* const*>(a.peer_out) : &local_out;
    const int nbases = a.world > 0 ? a.world : 1;
    const int hq_all = a.world > 0 ? a.world * a.Hq : a.Hq;       // heads of the destination tensor
    const int hq_off = a.world > 0 ? a.rank * a.Hq : 0;           // where this rank's heads start in it
    pdl_wait();          // partials are complete and visible once the attention grid has finished
#ifdef HOGATT_TIMELINE
    if (threadIdx.x == 0 && mcta < 128) g_mphase[a.debug_id % kTraceCalls][1][mcta] = global_timer_ns_();
#endif
    // (Running the whole merge once on stale data before the wait, nothing stored, so that its instructions are on the
    // SM when the wait ends: measured +0.1 ... +0.5 us per call, not kept.)
#pragma unroll 1
    for (int row = blockIdx.y * MW + warp; row < RPB; row += gridDim.y * MW) {
        const int gr = rb * RPB + row;
        if (gr >= a.rows_total) continue;
        const RowId id = decode_row(gr, a.G, a.S);
        const size_t offset = ((size_t)(id.w * hq_all + hq_off + hkv * a.G + id.g) * a.S + id.s) * Ev;
#pragma unroll 1
        for (int e0 = 0; e0 < Ev; e0 += 128)
#ifdef HOGATT_TIMELINE
            merge_partials_rows<T, NSTAT, KB>(a.ws_o, a.ws_m, a.ws_l, (size_t)u * a.parts_per_unit, RPB, Ev, row, a.parts_per_unit,
                                              count_of, bases, nbases, offset, lane, e0,
                                              (warp == 0 && mcta < 128) ? &g_mphase[a.debug_id % kTraceCalls][2][mcta] : nullptr);
#else
            merge_partials_rows<T, NSTAT, KB>(a.ws_o, a.ws_m, a.ws_l, (size_t)u * a.parts_per_unit, RPB, Ev, row, a.parts_per_unit,
                                              count_of, bases, nbases, offset, lane, e0);
#endif
    }
    HOGATT_SPAN_MAX(3);
#ifdef HOGATT_TIMELINE
    if (threadIdx.x == 0 && mcta < 128) g_mphase[a.debug_id % kTraceCalls][3][mcta] = global_timer_ns_();
    if (threadIdx.x == 0) atomicMax(&g_mtrace[a.debug_id % kTraceCalls][1], global_timer_ns_());
#endif
}

// Split-K merge for rows with MANY partials (kv heads sharded over GPUs: one unit cut into a partial per SM).  One CTA
// per output row, eight warps; warp w folds partials w, w + 8, ... exactly like merge_partials_rows does (its own
// maximum, denominator and weighted sum: one memory round trip for up to 192 partials per row), the eight results are
// combined through shared memory.  The one-warp-per-row kernel above needs a round trip per 24 partials.
constexpr int kWideWarps = 8;
template <class T, int WW = kWideWarps, int KP = 24>
__global__ void __launch_bounds__(WW * 32, (WW == 4 && KP == 16) ? 5 : 1) merge_wide_kernel(const __grid_constant__ KernelArgs a) {
    __shared__ float sm_m[WW], sm_l[WW];
    __shared__ float4 sm_o[WW][64];               // up to 256 output columns
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int u = blockIdx.x, row = blockIdx.y;
    const int rb = u / a.Hkv, hkv = u % a.Hkv;
    pdl_trigger();
    pdl_wait();
#ifdef HOGATT_TIMELINE
    if (threadIdx.x == 0) atomicMin(&g_mtrace[a.debug_id % kTraceCalls][0], global_timer_ns_());   // (here: the wait is over)
#endif
    const int units = a.row_blocks * a.Hkv;
    const int RPB = a.rows_per_block, Ev = a.Ev;
    const int gr = rb * RPB + row;
    if (gr >= a.rows_total) return;      // (uniform over the CTA)
    int count = 0;
    {
        const int TH = a.host_plan ? a.plan_tiles : __ldcg(a.header), ctas = a.host_plan ? a.plan_ctas : __ldcg(a.header + 1);
        int first = 0;
        if (TH > 0) unit_ctas(u, TH, (int64_t)units * TH, ctas, &first, &count);
    }
    const size_t slot0 = (size_t)u * a.parts_per_unit;
    // partials per warp per pass.  (Four warps x 16 under 102 registers make a CTA of 13 K registers, which fits on an
    // SM beside a resident attention CTA; with 24 per warp the kernel takes 168 registers.)
    constexpr int kPer = KP;
    float M = -INFINITY, L = 0.f;
    float4 acc[2] = {make_float4(0.f, 0.f, 0.f, 0.f), make_float4(0.f, 0.f, 0.f, 0.f)};     // columns lane*4 (+128)
#pragma unroll 1
    for (int p0 = warp; p0 < count; p0 += WW * kPer) {
        // this pass: partials p0, p0 + 8, ...; lane k holds the statistics of the k-th of them
        const int mine = p0 + lane * WW;
        const bool have = lane < kPer && mine < count;
        const float mp = have ? __ldcg(a.ws_m + (slot0 + mine) * RPB + row) : -INFINITY;
        const float lp = have ? __ldcg(a.ws_l + (slot0 + mine) * RPB + row) : 0.f;
        float4 x[kPer];
        const bool wide = Ev > 128;
#pragma unroll
        for (int k = 0; k < kPer; ++k) {             // (only the partials that exist: with 39 per row a warp has ten, not 24)
            const int p = p0 + k * WW;
            x[k] = (lane * 4 < Ev && p < count)
                       ? __ldcg(reinterpret_cast<const float4*>(a.ws_o + ((slot0 + p) * RPB + row) * Ev + lane * 4))
                       : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        float Mp = mp;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) Mp = fmaxf(Mp, __shfl_xor_sync(0xffffffffu, Mp, o));
        const float Mn = fmaxf(M, Mp);
        const float mu = Mn == -INFINITY ? 0.f : Mn;
        const float rescale = exp2f(M - mu);               // (M = -inf -> 0)
        const float w = have ? exp2f(mp - mu) : 0.f;
        float den = lp * w;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) den += __shfl_xor_sync(0xffffffffu, den, o);
        L = L * rescale + den;
        M = Mn;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            acc[h].x *= rescale;
            acc[h].y *= rescale;
            acc[h].z *= rescale;
            acc[h].w *= rescale;
        }
#pragma unroll
        for (int k = 0; k < kPer; ++k) {
            const float wk = __shfl_sync(0xffffffffu, w, k);
            const bool used = p0 + k * WW < count;   // a repeated last slot must not count twice
            acc[0].x = fmaf(used ? x[k].x : 0.f, wk, acc[0].x);
            acc[0].y = fmaf(used ? x[k].y : 0.f, wk, acc[0].y);
            acc[0].z = fmaf(used ? x[k].z : 0.f, wk, acc[0].z);
            acc[0].w = fmaf(used ? x[k].w : 0.f, wk, acc[0].w);
        }
        if (wide) {                                         // columns 128 .. 255: a second pass over the same partials
#pragma unroll 1
            for (int k = 0; k < kPer; ++k) {
                const int p = p0 + k * WW;
                if (p >= count) break;
                const float wk = __shfl_sync(0xffffffffu, w, k);
                if (128 + lane * 4 < Ev) {
                    const float4 y = __ldcg(reinterpret_cast<const float4*>(a.ws_o + ((slot0 + p) * RPB + row) * Ev + 128 + lane * 4));
                    acc[1].x = fmaf(y.x, wk, acc[1].x);
                    acc[1].y = fmaf(y.y, wk, acc[1].y);
                    acc[1].z = fmaf(y.z, wk, acc[1].z);
                    acc[1].w = fmaf(y.w, wk, acc[1].w);
                }
            }
        }
    }
    if (lane == 0) {
        sm_m[warp] = M;
        sm_l[warp] = L;
    }
    sm_o[warp][lane] = acc[0];
    sm_o[warp][32 + lane] = acc[1];
    __syncthreads();
    // every thread of the first two warps finishes four output columns
    if (warp < 2 && (warp * 128 + lane * 4) < Ev) {
        float Mx = sm_m[0];
#pragma unroll
        for (int k = 1; k < WW; ++k) Mx = fmaxf(Mx, sm_m[k]);
        const float mu = Mx == -INFINITY ? 0.f : Mx;
        float den = 0.f;
        float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int k = 0; k < WW; ++k) {
            const float f = sm_m[k] == -INFINITY ? 0.f : exp2f(sm_m[k] - mu);      // a warp without partials holds zeros
            const float4 y = sm_o[k][warp * 32 + lane];
            den = fmaf(sm_l[k], f, den);
            sum.x = fmaf(y.x, f, sum.x);
            sum.y = fmaf(y.y, f, sum.y);
            sum.z = fmaf(y.z, f, sum.z);
            sum.w = fmaf(y.w, f, sum.w);
        }
        const float inv = den > 0.f ? 1.f / den : 0.f;
        if (!(den > 0.f)) sum = make_float4(0.f, 0.f, 0.f, 0.f);
        const RowId id = decode_row(gr, a.G, a.S);
        T* const local_out = static_cast<T*>(a.out);
        const int nbases = a.world > 0 ? a.world : 1;
        const int hq_all = a.world > 0 ? a.world * a.Hq : a.Hq, hq_off = a.world > 0 ? a.rank * a.Hq : 0;
        const size_t offset = ((size_t)(id.w * hq_all + hq_off + hkv * a.G + id.g) * a.S + id.s) * Ev + warp * 128 + lane * 4;
        for (int b = 0; b < nbases; ++b)
            store4<T>((a.world > 0 ? static_cast<T*>(a.peer_out[b]) : local_out) + offset, sum.x * inv, sum.y * inv, sum.z * inv,
                      sum.w * inv);
    }
#ifdef HOGATT_TIMELINE
    if (threadIdx.x == 0) atomicMax(&g_mtrace[a.debug_id % kTraceCalls][1], global_timer_ns_());
#endif
}

// Completion exchange of the fused output all-gather: one warp, lane p talks to rank p.
//   1. bump this rank's call counter (device memory, so that a replayed CUDA graph still counts);
//   2. publish the new count into slot `rank` of every peer's flag array (system-scope release: the
//      merge kernel's peer stores, finished at the kernel boundary before this one, are visible first);
//   3. wait -- bounded -- until every peer has published at least the same count into OUR flag array.
// flags layout on every rank: int32[world] flags + int32 counter at index `world`.
// (Publishing from the tail of the kernel that stores the rows instead -- every CTA fences its peer stores at
// system scope and takes a ticket, the last one publishes, this kernel only waits -- was measured on two GPUs:
// 29.7 ... 32.8 us per call against 21 ... 23 with the exchange behind the kernel boundary; the per-CTA
// system-scope fences sit on the storing kernel's critical path.)
struct PeerFlags {
    int* f[HOGATT_MAX_PEERS];
};
__global__ void __launch_bounds__(32) gather_signal_kernel(const __grid_constant__ PeerFlags flags, int world, int rank,
                                                           int* status, int debug_id) {
    const int lane = threadIdx.x;
    int* mine = flags.f[rank];
    int epoch = 0;
#ifdef HOGATT_TIMELINE
    if (lane == 0) g_strace[debug_id % kTraceCalls][0] = global_timer_ns_();
#endif
    pdl_trigger();       // the next call's attention kernel may be scheduled (it waits for this grid before it reads or writes anything of this call's)
    pdl_wait();          // the rows are out: the storing kernel has completed and its stores are flushed
#ifdef HOGATT_TIMELINE
    if (lane == 0) g_strace[debug_id % kTraceCalls][1] = global_timer_ns_();
#endif
    if (lane == 0) epoch = atomicAdd(mine + world, 1) + 1;
    epoch = __shfl_sync(0xffffffffu, epoch, 0);
    if (lane < world) {
        // (the release store orders everything that happened before it -- the storing kernel's rows, complete and
        // flushed at the kernel boundary -- in front of the count; with an explicit system fence in front of it as
        // well, publishing took 3.3 us of a 20 us call on two GPUs, without it 1.8-2.3 us)
        asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(flags.f[lane] + rank), "r"(epoch) : "memory");
#ifdef HOGATT_TIMELINE
        if (lane == 0) g_strace[debug_id % kTraceCalls][2] = global_timer_ns_();
#endif
        const uint64_t t0 = global_timer_ns();
        while (true) {
            int seen;
            asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(seen) : "l"(mine + lane) : "memory");
            if (seen >= epoch) break;
            if (global_timer_ns() - t0 > g_wait_limit_ns) {
                if (status) atomicOr(status, STATUS_WAIT_PEER_TIMEOUT);
                break;
            }
            __nanosleep(100);
        }
    }
#ifdef HOGATT_TIMELINE
    __syncwarp();
    if (lane == 0) g_strace[debug_id % kTraceCalls][3] = global_timer_ns_();
#endif
}

// rq[f,w,h,s,:] = rope(q[w,h,s,:], cos[f,w,s,:], sin[f,w,s,:]).
// Replaces rope_kernel (src/rope.cuh:2-52), which uses one thread per channel and one CTA per row;
// here a thread produces a 16-byte chunk of a row from 16-byte loads.
template <class T>
__global__ void __launch_bounds__(128) rope_kernel(T* __restrict__ rq, const T* __restrict__ q,
                                                   const float* __restrict__ cosines,
                                                   const float* __restrict__ sines, int F, int W, int Hq, int S,
                                                   int E, int R) {
    write_rotated_queries<T>(q, rq, cosines, sines, F, W, Hq, S, E, R, blockIdx.x * blockDim.x + threadIdx.x,
                             gridDim.x * blockDim.x);
}

// The same for 16-bit types with the whole head rotated (R == E, E a multiple of 16): a thread owns one pair of
// 16-byte chunks (channels 8j.. and E/2 + 8j.., each the other's rotation partner) of one (f, w, s), keeps their four
// table chunks in registers and walks kRopeHeads query heads with them: per 32 output bytes two 16-byte loads
// instead of twelve.  Arithmetic and rounding are rotate_chunk's, so the bits are the same.
constexpr int kRopeHeads = 4;
template <class T>
__global__ void __launch_bounds__(128) rope_pairs_kernel(T* __restrict__ rq, const T* __restrict__ q,
                                                         const float* __restrict__ cosines, const float* __restrict__ sines,
                                                         int F, int W, int Hq, int S, int E) {
    const int pairs = E >> 4, half = E >> 1;
    const int item = blockIdx.x * blockDim.x + threadIdx.x;
    if (item >= F * W * S * pairs) return;
    const int j = item % pairs;
    int t = item / pairs;
    const int s = t % S;
    t /= S;
    const int w = t % W, f = t / W;
    const size_t tab = ((size_t)(f * W + w) * S + s) * E + 8 * j;
    float cl[8], sl[8], chh[8], shh[8];
    *reinterpret_cast<float4*>(cl) = *reinterpret_cast<const float4*>(cosines + tab);
    *reinterpret_cast<float4*>(cl + 4) = *reinterpret_cast<const float4*>(cosines + tab + 4);
    *reinterpret_cast<float4*>(sl) = *reinterpret_cast<const float4*>(sines + tab);
    *reinterpret_cast<float4*>(sl + 4) = *reinterpret_cast<const float4*>(sines + tab + 4);
    *reinterpret_cast<float4*>(chh) = *reinterpret_cast<const float4*>(cosines + tab + half);
    *reinterpret_cast<float4*>(chh + 4) = *reinterpret_cast<const float4*>(cosines + tab + half + 4);
    *reinterpret_cast<float4*>(shh) = *reinterpret_cast<const float4*>(sines + tab + half);
    *reinterpret_cast<float4*>(shh + 4) = *reinterpret_cast<const float4*>(sines + tab + half + 4);
    const int h0 = blockIdx.y * kRopeHeads;
    uint4 xl[kRopeHeads], xh[kRopeHeads];
#pragma unroll
    for (int k = 0; k < kRopeHeads; ++k) {
        const int h = min(h0 + k, Hq - 1);
        const T* row = q + ((size_t)(w * Hq + h) * S + s) * E + 8 * j;
        xl[k] = *reinterpret_cast<const uint4*>(row);
        xh[k] = *reinterpret_cast<const uint4*>(row + half);
    }
#pragma unroll
    for (int k = 0; k < kRopeHeads; ++k) {
        if (h0 + k >= Hq) break;
        const T* a = reinterpret_cast<const T*>(&xl[k]);
        const T* b = reinterpret_cast<const T*>(&xh[k]);
        uint4 lo, hi;
        uint32_t* ol = reinterpret_cast<uint32_t*>(&lo);
        uint32_t* oh = reinterpret_cast<uint32_t*>(&hi);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float rl[2], rh[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int c = 2 * i + e;
                const float av = Scalar<T>::to_float(a[c]), bv = Scalar<T>::to_float(b[c]);
                rl[e] = __fsub_rn(__fmul_rn(av, cl[c]), __fmul_rn(bv, sl[c]));
                rh[e] = __fadd_rn(__fmul_rn(bv, chh[c]), __fmul_rn(av, shh[c]));
            }
            ol[i] = pack2<T>(rl[0], rl[1]);
            oh[i] = pack2<T>(rh[0], rh[1]);
        }
        T* dst = rq + ((size_t)((f * W + w) * Hq + h0 + k) * S + s) * E + 8 * j;
        *reinterpret_cast<uint4*>(dst) = lo;
        *reinterpret_cast<uint4*>(dst + half) = hi;
    }
}

}  // namespace hogatt
