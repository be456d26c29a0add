// Tensor-core fragment attention for fp16 / bf16 with E == Ev in {64, 128}: the hot path.
//
// Two launch shapes of one kernel (template parameter CL, see the comment above the kernel): a persistent
// grid, one CTA per SM walking a contiguous range of KV tiles (hogatt_plan.h), partial results merged by
// merge_kernel; or thread-block clusters, one per (kv head, row block) unit, which merge by themselves
// through distributed shared memory.  Inside a CTA both are the same:
//   * warp 0 is the producer: it streams K and V tiles global -> shared with 1-D bulk async
//     copies (TMA engine) into a ring of NSTAGE stages, completion counted on mbarriers.  A tile
//     is a run of consecutive keys of one fragment and one
//     kv head, which is one contiguous byte run because fragments are [Hkv, rows, E] row-major.
//     (A tile is 128 keys at head size 128 and 256 keys at head size 64: 64 KiB per stage, 3 stages.)
//   * consumer warps each keep 16 query rows (one MMA m-tile) of the kv head resident -- ALL
//     workers and GQA heads of the head share every K/V tile, so KV is read from HBM once per
//     call -- and take a slice of every tile: S = Q K^T and O += P V with mma.sync m16n8k16,
//     fp32 accumulate, online softmax in base 2 in registers.  The per-fragment query RoPE is
//     done in the prologue of each fragment: all consumer threads rotate 16-byte chunks of the
//     un-rotated query with the cos/sin rows (rounded to the storage type first, as the
//     reference's rope kernel does before attention reads them, src/rope.cuh:43-45), stage them in
//     shared memory, and each warp pulls its MMA A-fragments from there with ldmatrix.
//   * where the CTA's share of a (kv head, row block) unit ends, the warps fold their private
//     (O, max, sum) together through shared memory and leave one partial in the workspace.
//
// Shared-memory layout of a K (or V) tile: 8 groups of GT consecutive keys; group g starts at
// g * (GT * row_bytes + 16).  The MMA "n" (QK^T) / "k" (PV) index does not run over consecutive
// keys but over the 8 groups at a fixed position i inside the group: key = g * GT + i.  The 16
// bytes of padding per group rotate the bank of equal chunks by one 16-byte unit per group, so
// the 8 row addresses of every ldmatrix phase fall into 8 different bank groups: no bank
// conflicts although the bulk copies land rows unswizzled.  A tile is 8 bulk copies of 4 KiB for K
// and 8 for V (issuing a copy costs the producer ~55 ns whatever its size, so copies are made large).
//
// The reference kernel (src/kernels/kernel_v21.cuh:28-316) assigns one (kv head, worker, token,
// split) to a CTA, keeps the GQA heads' queries and accumulators in registers/local memory,
// reduces dot products with 8-lane shuffles on CUDA cores and stages 32 rows per step with
// 16-byte cp.async; it re-reads the KV once per (worker, token).
#pragma once
#include "hogatt_device.cuh"

namespace hogatt {

template <int HD, int MT>
struct MmaCfg {
    // consumer warps.  Up to 8 warps per CTA may use 255 registers each; beyond that the register file only
    // gives 168, which spills the accumulators -- so one or two m-tiles run on 4 warps (four or two key
    // slices each).  (8 consumer warps for every shape were measured: 2-4 us slower per call.)
    static constexpr int NCW = (MT == 4) ? 8 : 4;
    static constexpr int NSLICE = NCW / MT;              // warps sharing one m-tile, each takes a slice of the keys
    static constexpr int GT = (HD == 128) ? 16 : 32;     // keys per group (one 4 KiB bulk copy)
    static constexpr int TILE = 8 * GT;                  // keys per stage
    static constexpr int ROWB = HD * 2;                  // bytes per key row
    static constexpr int GROUP_STRIDE = GT * ROWB + 16;
    static constexpr int KV_BYTES = 8 * GROUP_STRIDE;
    static constexpr int STAGE_BYTES = 2 * KV_BYTES;
    static constexpr int NSTAGE = 3;
    static constexpr int NT_S = GT / NSLICE;             // 8-key n-tiles per warp per stage
    static constexpr int NT_O = HD / 8;                  // output n-tiles
    static constexpr int KSTEPS = HD / 16;
    // Producer warps: warp 0, and with NPW == 2 also warp NCW + 1 (then warp 0 copies the K half of a tile,
    // the other the V half).  Issuing one bulk copy costs the issuing warp ~55 ns whatever its size, so one
    // producer needs 0.88 us for the 16 copies of a stage, which caps one SM at 74 GB/s; two producers lift
    // that to ~100 GB/s per SM.  With a CTA on every SM the chip's HBM gives each SM 44 GB/s, and the
    // second producer measured 0.5-1 us SLOWER per call there; it only pays when few SMs stream a lot.
    static constexpr int NPW = 1;
    // Helper warp (decode-sized query blocks only): writes the rotated-query side output, so that neither the
    // producer (whose copies would stall behind those loads and stores) nor the consumers (whose first tile would)
    // has to.  Ten warps would cut the register budget of the 64-row variant, which writes it with its consumers.
    static constexpr int NHW = (MT <= 2) ? 1 : 0;
    static constexpr int THREADS = (NCW + NPW + NHW) * 32;
    static constexpr int RPB = 16 * MT;                  // query rows per CTA
    static constexpr int SLOT_FLOATS = NT_O * 4 * 32;    // one warp's accumulators
    static constexpr int QPITCH = ROWB + 16;             // bytes per staged query row (padding: conflict-free ldmatrix)
    static constexpr int QBYTES = RPB * QPITCH;
    // Second query tile (+ one visibility limit per row): a CTA whose tile range runs on into a second fragment
    // or unit stages that segment's rotated queries at kernel start too, while ordinary loads still take one
    // quick round trip -- in the middle of the stream they queue behind megabytes of bulk copies.  Where the
    // For 16- and 32-row blocks; with 64 rows the shared memory has no room for it and every segment is staged
    // when it is reached.  (32 rows: a 20-byte spill outside the streaming loop; measured -0.1 us at GQA 5.)
    static constexpr int Q2BYTES = (MT <= 2) ? QBYTES + RPB * 4 : 0;
    // cluster variant: what a CTA leaves in its own shared memory for the cluster-wide merge
    static constexpr int OPITCH = HD + 8;                // floats per partial row (padding: conflict-free float2 stores)
    static constexpr int CL_PART_FLOATS = 16 * OPITCH;   // one warp's 16 rows
    static constexpr int CL_STAT = NCW * CL_PART_FLOATS; // float offset of the row maxima [NCW][16], sums follow
    static constexpr int CL_ACC = CL_STAT + 2 * NCW * 16;        // merge scratch [tasks <= RPB][HD]
    static constexpr int CL_DEN = CL_ACC + RPB * HD;             // [tasks]
    static constexpr int CL_FLOATS = CL_DEN + RPB;
    static_assert(CL_FLOATS * 4 <= NSTAGE * STAGE_BYTES, "cluster merge scratch must fit in the stage ring");
    static_assert(NT_S >= 2 && NT_S % 2 == 0, "a warp's slice must hold whole k16 steps");
    static_assert(NCW * SLOT_FLOATS * 4 <= STAGE_BYTES, "fold scratch must fit in one stage");
    static_assert(NT_O % NSLICE == 0, "output columns must split evenly over the slices");
};

template <int HD, int MT>
__host__ __device__ inline size_t mma_smem_bytes(int F) {
    using C = MmaCfg<HD, MT>;
    return 128 /* alignment slack */ + (size_t)C::NSTAGE * C::STAGE_BYTES + C::QBYTES + C::Q2BYTES +
           (size_t)C::NCW * 32 * 4 * 4 /* stats */ + (2 * C::NSTAGE + 1) * 8 /* barriers */ + 16 /* abort flag */ +
           ((size_t)2 * F + 1) * 4;
}

// rotate_chunk for tables or rotary sizes the 16-byte path cannot take (rotary_dim not a multiple of 16,
// tables not 16-byte aligned): eight channels one by one.  Rare, and kept out of line.
template <class T>
__device__ __noinline__ uint4 rotate_chunk_by_channel(const T* q, const float* c, const float* s, int ch, int R) {
    uint4 v;
    uint32_t* o32 = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
    for (int k = 0; k < 4; ++k)
        o32[k] = pack2<T>(rope_channel<T>(q, c, s, ch * 8 + 2 * k, R), rope_channel<T>(q, c, s, ch * 8 + 2 * k + 1, R));
    return v;
}

// Destinations of a finished output row: this rank's `out`, or (fused all-gather) the full-size output of
// every rank at this rank's head offset.
template <class T>
struct OutputTargets {
    T* const* bases;
    T* local;
    int nbases, hq_all, hq_off;
    __device__ __forceinline__ explicit OutputTargets(const KernelArgs& a) : local(static_cast<T*>(a.out)) {
        nbases = a.world > 0 ? a.world : 1;
        hq_all = a.world > 0 ? a.world * a.Hq : a.Hq;
        hq_off = a.world > 0 ? a.rank * a.Hq : 0;
        bases = a.world > 0 ? reinterpret_cast<T* const*>(a.peer_out) : nullptr;
    }
    __device__ __forceinline__ T* base(int b) const { return bases ? bases[b] : local; }
    // element offset of row (w, local head hq, s)
    __device__ __forceinline__ size_t row_offset(int w, int hq, int s, int S, int Ev) const {
        return ((size_t)(w * hq_all + hq_off + hq) * S + s) * Ev;
    }
};

// Rows of fragment f that a query may see at all: under a device plan vis[f] is exact already; under a host plan
// vis[f] is only the host's bound, and the true length comes from the tensors' extent and the device-side lengths.
__device__ __forceinline__ int visible_length(const KernelArgs& a, int f, const int* vis) {
    int v = vis[f];
    if (a.host_plan && a.flen) v = min(v, a.flen[f]);
    return v;
}

// CL = false: persistent grid over balanced tile ranges, partials to the workspace, merge_kernel follows.
// CL = true : launched in thread-block clusters, one cluster per (kv head, row block) unit; CTA `rank`
//             of the cluster takes tiles [rank*TH/CS, (rank+1)*TH/CS) of the unit; every warp leaves its
//             private (O, max, sum) in its CTA's shared memory, and after a cluster barrier CTA `rank`
//             merges rows rank, rank+CS, ... of the block over ALL warps of ALL CTAs through distributed
//             shared memory and stores the final rows: no workspace traffic, no second kernel.
template <class T, int HD, int MT, bool CL>
__global__ void __launch_bounds__(MmaCfg<HD, MT>::THREADS, 1)
mma_attention_kernel(const __grid_constant__ KernelArgs a, const int use_evict_first) {
    using C = MmaCfg<HD, MT>;
    extern __shared__ unsigned char smem_dyn[];
    unsigned char* base = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 127) & ~(uintptr_t)127);
    unsigned char* stages = base;
    unsigned char* qtile = stages + (size_t)C::NSTAGE * C::STAGE_BYTES;                     // [RPB][QPITCH]
    unsigned char* qtile2 = qtile + C::QBYTES;                                              // [RPB][QPITCH] + int[RPB]
    float* stats = reinterpret_cast<float*>(qtile2 + C::Q2BYTES);                           // [NCW][32][4]
    uint64_t* bars = reinterpret_cast<uint64_t*>(stats + C::NCW * 32 * 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2 * C::NSTAGE + 1);
    int* vis = const_cast<int*>(abort_flag) + 4;
    int* pre = vis + a.F;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    HOGATT_TL_DECL;
    HOGATT_TL(warp == 0 ? 0 : 1, 1);
    HOGATT_SPAN_MIN(0);
    if (tid == 0) HOGATT_TRACE(a.debug_id, 0);
#ifdef HOGATT_TIMELINE
    if (tid == 0) {
        g_cta_t[0][blockIdx.x] = global_timer_ns_();
        unsigned int smid;
        asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
        g_cta_sm[blockIdx.x] = smid;
    }
#endif
    const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * C::NSTAGE, cbar = full0 + 16 * C::NSTAGE;
    const uint32_t stage0 = smem_u32(stages);

    if (tid == 0) {
        for (int s = 0; s < C::NSTAGE; ++s) {
            mbar_init(full0 + 8 * s, C::NPW);
            mbar_init(empty0 + 8 * s, C::NCW);
        }
        mbar_init(cbar, C::NCW);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_proxy_async_smem();
    }
    // Programmatic dependent launch: this grid may have been scheduled while the stream's preceding kernel is
    // still running.  `waited` says whether this thread has passed griddepcontrol.wait, i.e. may touch global
    // memory that earlier work writes or reads (everything except the K/V rows of "stable" fragments).
    const bool is_helper = C::NHW != 0 && warp == C::NCW + C::NPW;
    const bool is_producer = warp == 0 || (warp > C::NCW && !is_helper);
    bool waited;
    if (a.host_plan) {
        // The tile plan comes from the kernel arguments: nothing is read from device memory before the first
        // K/V copy.  Every thread waits where it first needs global memory that earlier work may write: the
        // consumers in their first fragment prologue (queries, tables, locations), the producer when it reaches a
        // tile that it may not fetch early (or has filled the ring and sent the rest of its stable tiles to L2).
        if (warp == 0) host_tile_prefix(a, C::TILE, vis, pre);
        __syncthreads();                         // barriers and plan are visible
        waited = false;
    } else {
        pdl_wait();      // everything above touched only this CTA's shared memory
        pdl_trigger();   // the merge kernel may take its place on the SMs now; it waits for this grid itself
        build_tile_prefix(a, C::TILE, vis, pre);     // ends with __syncthreads(): barriers are visible too
        waited = true;
        if (tid == 32) HOGATT_TRACE(a.debug_id, 1);
    }
    if (warp <= 1) HOGATT_TL(warp, 2);

    const int TH = pre[a.F];
    const int units = a.row_blocks * a.Hkv;
    const int64_t N = (int64_t)units * TH;
    const int ctas = CL ? (int)gridDim.x : (a.host_plan ? a.plan_ctas : aligned_ctas(pre, a.F, units, gridDim.x));
    const int CS = CL ? (int)cluster_nctarank() : 1, crank = CL ? (int)cluster_ctarank() : 0;
    if (!CL && !a.host_plan && blockIdx.x == 0 && tid == 0) {      // (host plan: the merge kernel has both as arguments)
        a.header[0] = TH;
        a.header[1] = ctas;
    }
    // The rotated-query output is a side product every CTA writes a share of.  When it is small (a few
    // 16-byte chunks per thread: decode) the helper warp writes it, which keeps those loads and stores off the
    // consumers' start-up path and off the producer's copy stream.  When it is large (many query tokens) the
    // consumer threads write it after their first fragment prologue, while the first K/V tile is still in flight,
    // with far more loads in flight than one warp could keep.
    const bool want_rq = a.rq != nullptr && a.cos != nullptr;
    const bool rq_by_helper =
        C::NHW != 0 && want_rq && (int64_t)a.F * a.W * a.Hq * a.S * (HD / 8) <= (int64_t)8 * gridDim.x * 32;
    const bool rq_by_consumers = want_rq && !rq_by_helper;
    if ((int)blockIdx.x >= ctas) {
        if (!waited) pdl_wait();
        if (rq_by_helper && is_helper)
            write_rotated_queries<T>(a.q, a.rq, a.cos, a.sin, a.F, a.W, a.Hq, a.S, HD, a.R, blockIdx.x * 32 + lane,
                                     gridDim.x * 32);
        if (rq_by_consumers && warp > 0 && warp <= C::NCW)
            write_rotated_queries<T>(a.q, a.rq, a.cos, a.sin, a.F, a.W, a.Hq, a.S, HD, a.R,
                                     blockIdx.x * (C::NCW * 32) + tid - 32, gridDim.x * (C::NCW * 32));
        return;
    }
    if (warp <= 1) HOGATT_TL(warp, 3);

    int64_t t0, t1;
    if constexpr (CL) {
        const int64_t ubase = (int64_t)(blockIdx.x / CS) * TH;
        t0 = ubase + (int64_t)crank * TH / CS;
        t1 = ubase + (int64_t)(crank + 1) * TH / CS;
    } else {
        t0 = cta_first_tile(blockIdx.x, N, ctas);
        t1 = cta_first_tile(blockIdx.x + 1, N, ctas);
    }

    if (is_helper) {
        if (!waited) pdl_wait();
        if (rq_by_helper)
            write_rotated_queries<T>(a.q, a.rq, a.cos, a.sin, a.F, a.W, a.Hq, a.S, HD, a.R, blockIdx.x * 32 + lane,
                                     gridDim.x * 32);
        if constexpr (CL) {
            cluster_sync_all();
            cluster_sync_all();
        }
        return;
    }

    // =====================================================================================
    // Producer warp
    // =====================================================================================
    if (is_producer) {
        constexpr int COPIES = 16 / C::NPW;              // bulk copies per producer warp per stage (8 K groups + 8 V groups in all)
        const int copy0 = warp == 0 ? 0 : COPIES;
        uint64_t policy = 0;
        if (use_evict_first & 1) policy = l2_policy_evict_first();
        int64_t u = CL ? (int64_t)(blockIdx.x / CS) : t0 / TH;
        int j = (int)(t0 - u * TH), fscan = 0, it = 0;
        bool ok = true;
#pragma unroll 1
        for (int64_t t = t0; t < t1 && ok; ++t, ++it) {
            while (j >= pre[fscan + 1]) ++fscan;
            const int f = fscan;
            const int hkv = (int)(u % a.Hkv);
            const int tok0 = (j - pre[f]) * C::TILE;
            const int ntok = min(C::TILE, vis[f] - tok0);
            const int stage = it % C::NSTAGE;
            const uint32_t phase = (uint32_t)(it / C::NSTAGE) & 1u;
            if (!waited && (it >= C::NSTAGE || f >= a.stable_fragments)) {
                // The ring is full, or the next tile belongs to a fragment the stream's earlier work may still write.
                // (Asking for the CTA's further stable tiles to be brought into L2 here was measured and dropped: the
                // prefetches queue in front of the query loads that follow the wait, +0.5 us per call.)
                pdl_wait();                      // from here on: fragments that earlier work of the stream may have written
                waited = true;
                if (tid == 0) HOGATT_TRACE(a.debug_id, 5);
            }
            ok = mbar_wait_bounded(empty0 + 8 * stage, phase ^ 1u, abort_flag, a.status, STATUS_WAIT_EMPTY_TIMEOUT);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            const uint32_t fullb = full0 + 8 * stage;
            if (lane == 0) mbar_arrive_expect_tx(fullb, (uint32_t)ntok * C::ROWB * (2u / C::NPW));
            __syncwarp();
            if (lane < COPIES) {
                const int g = (copy0 + lane) & 7;
                const bool is_v = copy0 + lane >= 8;
                const int tg = min(C::GT, ntok - g * C::GT);
                if (tg > 0) {
                    const unsigned char* src = static_cast<const unsigned char*>(is_v ? a.ft.e[f].v : a.ft.e[f].k) +
                                               ((size_t)hkv * a.ft.e[f].rows + tok0 + g * C::GT) * C::ROWB;
                    const uint32_t dst = stage0 + stage * C::STAGE_BYTES + (is_v ? C::KV_BYTES : 0) + g * C::GROUP_STRIDE;
                    if (use_evict_first & 1)
                        bulk_load_hint(dst, src, (uint32_t)tg * C::ROWB, fullb, policy);
                    else
                        bulk_load(dst, src, (uint32_t)tg * C::ROWB, fullb);
                }
            }
            HOGATT_TL(0, 100 + it);
            if (tid == 0 && it == 0) HOGATT_TRACE(a.debug_id, 4);
            if (++j == TH) {
                j = 0;
                ++u;
                fscan = 0;
            }
        }
        if (!waited) pdl_wait();
        if (tid == 0) HOGATT_TRACE(a.debug_id, 6);
        // Do not leave while copies may still be landing in this CTA's shared memory.
        if (lane == 0) {
            const int pending = min(it, C::NSTAGE);
            for (int k = it - pending; k < it; ++k)
                mbar_wait_bounded(full0 + 8 * (k % C::NSTAGE), (uint32_t)(k / C::NSTAGE) & 1u, abort_flag, a.status,
                                  STATUS_DRAIN_TIMEOUT);
        }
        HOGATT_SPAN_MAX(1);
        if constexpr (CL) {
            cluster_sync_all();      // partials of every CTA are in place
            cluster_sync_all();      // nobody reads this CTA's shared memory any more
        }
        return;
    }

    // =====================================================================================
    // Consumer warps
    // =====================================================================================
    const int cw = warp - 1;
    const int mt = cw % MT, slice = cw / MT;
    const int quad = lane >> 2, qlane = lane & 3;
    const int row_a = mt * 16 + quad, row_b = row_a + 8;     // rows inside the block
    const T* __restrict__ q = static_cast<const T*>(a.q);

    float o[C::NT_O][4];
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
    uint32_t qf[C::KSTEPS][4];
    int lim_a = 0, lim_b = 0, wlim = 0;      // wlim: the largest limit of any row of this warp
    RowId id_a = {0, 0, 0}, id_b = {0, 0, 0};
    bool valid_a = false, valid_b = false;
    uint32_t cphase = 0;

    auto consumer_sync = [&]() -> bool {
        __syncwarp();
        if (lane == 0) mbar_arrive(cbar);
        const bool ok = mbar_wait_bounded(cbar, cphase, abort_flag, a.status, STATUS_WAIT_SYNC_TIMEOUT);
        cphase ^= 1u;
        return __all_sync(0xffffffffu, ok);
    };

    int64_t u = CL ? (int64_t)(blockIdx.x / CS) : t0 / TH;
    int j = (int)(t0 - u * TH), fscan = 0, it = 0, cur_u = -1, cur_f = -1, hkv = 0, rb = 0;
    int pre_u = -1, pre_f = -1;          // the segment whose queries sit in the second tile
#pragma unroll 1
    for (int64_t t = t0; t < t1; ++t, ++it) {
        if ((int)u != cur_u) {
            cur_u = (int)u;
            cur_f = -1;
            fscan = 0;
            rb = cur_u / a.Hkv;
            hkv = cur_u % a.Hkv;
            const int gra = rb * C::RPB + row_a, grb = rb * C::RPB + row_b;
            valid_a = gra < a.rows_total;
            valid_b = grb < a.rows_total;
            id_a = decode_row(valid_a ? gra : 0, a.G, a.S);
            id_b = decode_row(valid_b ? grb : 0, a.G, a.S);
            m_a = m_b = -INFINITY;
            l_a = l_b = 0.f;
#pragma unroll
            for (int n = 0; n < C::NT_O; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
        }
        while (j >= pre[fscan + 1]) ++fscan;
        const int f = fscan;
        if (f != cur_f) {
            cur_f = f;
            if (!waited) {
                pdl_wait();
                waited = true;
                if (tid == 32) HOGATT_TRACE(a.debug_id, 1);
                // Only now may the next kernel of the stream be scheduled behind this grid (it is, once every CTA has
                // said so): whatever it does before its own wait can then overlap with this call's kernels only,
                // never with work that was enqueued before this call.
                pdl_trigger();
            }
            // ---- per-fragment prologue ----------------------------------------------------------
            // All consumer threads rotate the block's query rows for this fragment (16-byte chunks,
            // every load independent: one memory round trip), round them to the storage type and
            // stage them in shared memory; each warp then pulls its MMA A-fragments with ldmatrix.
            const int vf = visible_length(a, f, vis);
            const unsigned char* qsrc = qtile;
            if (C::Q2BYTES != 0 && pre_u == cur_u && pre_f == f) {
                // staged at kernel start: nothing to load (the tile has been complete since the second
                // barrier of the first prologue, and nobody writes it again)
                const int* qlim2 = reinterpret_cast<const int*>(qtile2 + C::QBYTES);
                qsrc = qtile2;
                lim_a = qlim2[row_a];
                lim_b = qlim2[row_b];
                pre_u = -1;
            } else {
                const int loc_a = valid_a ? a.loc[(f * a.W + id_a.w) * a.S + id_a.s] : vf;
                const int loc_b = valid_b ? a.loc[(f * a.W + id_b.w) * a.S + id_b.s] : vf;
                // the segment after this one, if the CTA's range reaches it (first prologue only)
                int nseg = 1, u2 = 0, f2 = 0;
                if (C::Q2BYTES != 0 && it == 0) {
                    const int64_t seg_end = u * TH + pre[f + 1];
                    if (seg_end < t1) {
                        int j2 = pre[f + 1];
                        u2 = cur_u;
                        if (j2 >= TH) {
                            j2 = 0;
                            ++u2;
                        }
                        f2 = 0;
                        while (j2 >= pre[f2 + 1]) ++f2;
                        nseg = 2;
                        pre_u = u2;
                        pre_f = f2;
                    }
                }
                if (it != 0 && !consumer_sync()) break;        // everyone is done with the previous query tile (there is none at the start)
                if (warp == 1) HOGATT_TL(1, 20);
#pragma unroll 1
                for (int seg = 0; seg < nseg; ++seg) {
                    constexpr int CPR = HD / 8;                                    // 16-byte chunks per row
                    constexpr int NCHUNK = C::RPB * CPR;
                    constexpr int ITEMS = (NCHUNK + C::NCW * 32 - 1) / (C::NCW * 32);   // chunks per thread
                    const int sf = seg ? f2 : f, su = seg ? u2 : cur_u;
                    const int srb = su / a.Hkv, shkv = su % a.Hkv;
                    unsigned char* dst = seg ? qtile2 : qtile;
                    const bool chunked = a.cos == nullptr || chunked_rope_ok(a.cos, a.sin, a.R, HD);
                    const int ctid = tid - 32;
                    uint4 val[ITEMS];
                    bool live[ITEMS];
#pragma unroll
                    for (int k = 0; k < ITEMS; ++k) {          // all loads of all chunks are issued before any is used
                        const int item = ctid + k * (C::NCW * 32);
                        const int r = item / CPR, ch = item % CPR;
                        const int gr = srb * C::RPB + r;
                        live[k] = item < NCHUNK && gr < a.rows_total;
                        const RowId id = decode_row(live[k] ? gr : 0, a.G, a.S);
                        const int hq = shkv * a.G + id.g;
                        if (a.cos == nullptr) {
                            val[k] = *reinterpret_cast<const uint4*>(
                                q + ((size_t)((sf * a.W + id.w) * a.Hq + hq) * a.S + id.s) * HD + ch * 8);
                        } else {
                            const T* qrow = q + ((size_t)(id.w * a.Hq + hq) * a.S + id.s) * HD;
                            const size_t tab = ((size_t)(sf * a.W + id.w) * a.S + id.s) * a.R;
                            val[k] = chunked ? rotate_chunk<T>(qrow, a.cos + tab, a.sin + tab, ch, a.R)
                                             : rotate_chunk_by_channel<T>(qrow, a.cos + tab, a.sin + tab, ch, a.R);
                        }
                    }
                    if (seg && ctid < C::RPB) {                // visibility limits of the pre-staged segment
                        const int gr = srb * C::RPB + ctid;
                        const int v2 = visible_length(a, sf, vis);
                        int lim = v2;
                        if (gr < a.rows_total) {
                            const RowId id = decode_row(gr, a.G, a.S);
                            lim = min(a.loc[(sf * a.W + id.w) * a.S + id.s], v2 - 1) + 1;
                        }
                        reinterpret_cast<int*>(qtile2 + C::QBYTES)[ctid] = lim;
                    }
#pragma unroll
                    for (int k = 0; k < ITEMS; ++k) {
                        const int item = ctid + k * (C::NCW * 32);
                        const int r = item / CPR, ch = item % CPR;
                        if (item < NCHUNK)
                            *reinterpret_cast<uint4*>(dst + r * C::QPITCH + ch * 16) = live[k] ? val[k] : make_uint4(0u, 0u, 0u, 0u);
                    }
                }
                if (warp == 1) HOGATT_TL(1, 21);
                if (!consumer_sync()) break;                   // the query tile is complete
                if (warp == 1) HOGATT_TL(1, 22);
                if (tid == 32 && it == 0) HOGATT_TRACE(a.debug_id, 7);
                lim_a = valid_a ? min(loc_a, vf - 1) + 1 : vf;
                lim_b = valid_b ? min(loc_b, vf - 1) + 1 : vf;
            }
            wlim = max(lim_a, lim_b);
#pragma unroll
            for (int sh = 16; sh > 0; sh >>= 1) wlim = max(wlim, __shfl_xor_sync(0xffffffffu, wlim, sh));
            {
                const uint32_t qaddr = smem_u32(qsrc) + (mt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * C::QPITCH + (lane >> 4) * 16;
#pragma unroll
                for (int kk = 0; kk < C::KSTEPS; ++kk)
                    ldmatrix_x4(qaddr + kk * 32, qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3]);
            }
            if (rq_by_consumers && it == 0)
                write_rotated_queries<T>(a.q, a.rq, a.cos, a.sin, a.F, a.W, a.Hq, a.S, HD, a.R,
                                         blockIdx.x * (C::NCW * 32) + tid - 32, gridDim.x * (C::NCW * 32));
            if (warp == 1) HOGATT_TL(1, 10 + f);
        }
        const int tok0 = (j - pre[f]) * C::TILE;
        const int ntok = min(C::TILE, vis[f] - tok0);
        const int stage = it % C::NSTAGE;
        const uint32_t phase = (uint32_t)(it / C::NSTAGE) & 1u;
        const uint32_t kb = stage0 + stage * C::STAGE_BYTES, vb = kb + C::KV_BYTES;

        bool ok = mbar_wait_bounded(full0 + 8 * stage, phase, abort_flag, a.status, STATUS_WAIT_FULL_TIMEOUT);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        if (warp == 1) HOGATT_TL(1, 100 + it);
#ifdef HOGATT_TIMELINE
        if (warp == 1 && lane == 0 && it == 0) g_cta_t[1][blockIdx.x] = global_timer_ns_();
#endif
        if (tid == 32 && it == 0) HOGATT_TRACE(a.debug_id, 2);
#ifdef HOGATT_EXPERIMENT
        if (use_evict_first & 2) {           // stream only: hand the stage straight back (results are garbage)
            __syncwarp();
            if (lane == 0) mbar_arrive(empty0 + 8 * stage);
            if (++j == TH) {
                j = 0;
                ++u;
            }
            continue;
        }
#endif

        const int i0 = slice * C::NT_S;      // first in-group position of this warp's slice
        // Keys from `nvalid` on are masked for every row of this warp: their probabilities are exactly zero, but
        // 0 * NaN would poison the sums, and their V rows may hold anything -- past the end of a short tile the
        // copy wrote nothing, and under a host plan rows between a fragment's true length and the host's bound
        // are fetched as they are.  Make those V rows (of this warp's own slice) finite.
        const int nvalid = min(ntok, wlim - tok0);
        if (nvalid < C::TILE) {
            unsigned char* vgen = stages + (size_t)stage * C::STAGE_BYTES + C::KV_BYTES;
#pragma unroll 1
            for (int r = 0; r < 8 * C::NT_S; ++r) {
                const int g = r & 7, i = i0 + (r >> 3);
                if (g * C::GT + i >= nvalid && lane < C::ROWB / 16)
                    *reinterpret_cast<int4*>(vgen + g * C::GROUP_STRIDE + i * C::ROWB + lane * 16) = make_int4(0, 0, 0, 0);
            }
            __syncwarp();
        }

        // ---- S = Q K^T for this warp's keys ----
        float sc[C::NT_S][4];
#pragma unroll
        for (int ii = 0; ii < C::NT_S; ++ii) {
            sc[ii][0] = sc[ii][1] = sc[ii][2] = sc[ii][3] = 0.f;
            const uint32_t rowaddr = kb + (lane & 7) * C::GROUP_STRIDE + (i0 + ii) * C::ROWB + (lane >> 3) * 16;
#pragma unroll
            for (int k2 = 0; k2 < C::KSTEPS / 2; ++k2) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4(rowaddr + k2 * 64, b0, b1, b2, b3);
                mma_16816<T>(sc[ii], qf[2 * k2], b0, b1);
                mma_16816<T>(sc[ii], qf[2 * k2 + 1], b2, b3);
            }
        }

        // ---- visibility mask, online softmax (base 2) ----
        const int tile_end = tok0 + C::TILE;
        const bool need_mask = __any_sync(0xffffffffu, tile_end > lim_a || tile_end > lim_b);
        float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
        for (int ii = 0; ii < C::NT_S; ++ii) {
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                float xa = sc[ii][c] * a.l2scale, xb = sc[ii][2 + c] * a.l2scale;
                if (need_mask) {
                    const int key = tok0 + (qlane * 2 + c) * C::GT + i0 + ii;
                    if (key >= lim_a) xa = -INFINITY;
                    if (key >= lim_b) xb = -INFINITY;
                }
                sc[ii][c] = xa;
                sc[ii][2 + c] = xb;
                mx_a = fmaxf(mx_a, xa);
                mx_b = fmaxf(mx_b, xb);
            }
        }
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
        const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
        const float mu_a = (mn_a == -INFINITY) ? 0.f : mn_a, mu_b = (mn_b == -INFINITY) ? 0.f : mn_b;
        const float al_a = exp2f(m_a - mu_a), al_b = exp2f(m_b - mu_b);
        m_a = mn_a;
        m_b = mn_b;
        float ps_a = 0.f, ps_b = 0.f;
#pragma unroll
        for (int ii = 0; ii < C::NT_S; ++ii) {
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                sc[ii][c] = exp2f(sc[ii][c] - mu_a);
                sc[ii][2 + c] = exp2f(sc[ii][2 + c] - mu_b);
                ps_a += sc[ii][c];
                ps_b += sc[ii][2 + c];
            }
        }
        l_a = l_a * al_a + ps_a;     // per-thread share of the row sum; lanes of a quad are added at the fold
        l_b = l_b * al_b + ps_b;
        if (__any_sync(0xffffffffu, al_a != 1.f || al_b != 1.f)) {
#pragma unroll
            for (int n = 0; n < C::NT_O; ++n) {
                o[n][0] *= al_a;
                o[n][1] *= al_a;
                o[n][2] *= al_b;
                o[n][3] *= al_b;
            }
        }

        // ---- O += P V ----
#pragma unroll
        for (int ks = 0; ks < C::NT_S / 2; ++ks) {
            uint32_t pa[4];
            pa[0] = pack2<T>(sc[2 * ks][0], sc[2 * ks][1]);
            pa[1] = pack2<T>(sc[2 * ks][2], sc[2 * ks][3]);
            pa[2] = pack2<T>(sc[2 * ks + 1][0], sc[2 * ks + 1][1]);
            pa[3] = pack2<T>(sc[2 * ks + 1][2], sc[2 * ks + 1][3]);
            const uint32_t rowaddr =
                vb + (lane & 7) * C::GROUP_STRIDE + (i0 + 2 * ks + ((lane >> 3) & 1)) * C::ROWB + (lane >> 4) * 16;
#pragma unroll
            for (int jj = 0; jj < C::NT_O / 2; ++jj) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4_trans(rowaddr + jj * 32, b0, b1, b2, b3);
                mma_16816<T>(o[2 * jj], pa, b0, b1);
                mma_16816<T>(o[2 * jj + 1], pa, b2, b3);
            }
        }

        if (warp == 1) HOGATT_TL(1, 500 + it);
        // ---- end of this CTA's share of the unit: fold the warps together, leave a partial ----
        const bool last = (j == TH - 1) || (t == t1 - 1);
        bool wrote_scratch = false;
        if (!CL && last) {
            l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
            l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
            l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
            l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
            // Every warp parks its accumulators and statistics in this stage's buffer (it is still
            // owned by the consumers); then each warp combines, for its m-tile, ITS share of the
            // output columns over all slices and writes that share of the partial to the workspace.
            float* scratch = reinterpret_cast<float*>(stages + (size_t)stage * C::STAGE_BYTES);
            if (!consumer_sync()) break;                      // every warp is done reading this stage's K/V
            {
                float* dst = scratch + (size_t)(slice * MT + mt) * C::SLOT_FLOATS;
#pragma unroll
                for (int n = 0; n < C::NT_O; ++n)
#pragma unroll
                    for (int c = 0; c < 4; ++c) dst[(n * 4 + c) * 32 + lane] = o[n][c];
                *reinterpret_cast<float4*>(stats + ((slice * MT + mt) * 32 + lane) * 4) = make_float4(m_a, m_b, l_a, l_b);
                wrote_scratch = true;
            }
            if (!consumer_sync()) break;
            float fa[C::NSLICE], fb[C::NSLICE];
            float M_a = -INFINITY, M_b = -INFINITY, L_a = 0.f, L_b = 0.f;
            {
                float4 st[C::NSLICE];
#pragma unroll
                for (int sl = 0; sl < C::NSLICE; ++sl) {
                    st[sl] = *reinterpret_cast<const float4*>(stats + ((sl * MT + mt) * 32 + lane) * 4);
                    M_a = fmaxf(M_a, st[sl].x);
                    M_b = fmaxf(M_b, st[sl].y);
                }
                const float ua = (M_a == -INFINITY) ? 0.f : M_a, ub = (M_b == -INFINITY) ? 0.f : M_b;
#pragma unroll
                for (int sl = 0; sl < C::NSLICE; ++sl) {
                    fa[sl] = exp2f(st[sl].x - ua);
                    fb[sl] = exp2f(st[sl].y - ub);
                    L_a += st[sl].z * fa[sl];
                    L_b += st[sl].w * fb[sl];
                }
            }
            int first, count;
            unit_ctas(u, TH, N, ctas, &first, &count);
            const size_t slot = (size_t)u * a.parts_per_unit + (blockIdx.x - first);
            constexpr int NSHARE = C::NT_O / C::NSLICE;       // output n-tiles this warp combines
            float* wo_a = a.ws_o + (slot * C::RPB + row_a) * HD + qlane * 2;
            float* wo_b = a.ws_o + (slot * C::RPB + row_b) * HD + qlane * 2;
#pragma unroll
            for (int nn = 0; nn < NSHARE; ++nn) {
                const int n = slice * NSHARE + nn;
                float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int sl = 0; sl < C::NSLICE; ++sl) {
                    const float* src = scratch + (size_t)(sl * MT + mt) * C::SLOT_FLOATS + (n * 4) * 32 + lane;
                    acc[0] = fmaf(src[0], fa[sl], acc[0]);
                    acc[1] = fmaf(src[32], fa[sl], acc[1]);
                    acc[2] = fmaf(src[64], fb[sl], acc[2]);
                    acc[3] = fmaf(src[96], fb[sl], acc[3]);
                }
                *reinterpret_cast<float2*>(wo_a + n * 8) = make_float2(acc[0], acc[1]);
                *reinterpret_cast<float2*>(wo_b + n * 8) = make_float2(acc[2], acc[3]);
            }
            if (slice == 0 && qlane == 0) {
                a.ws_m[slot * C::RPB + row_a] = M_a;
                a.ws_m[slot * C::RPB + row_b] = M_b;
                a.ws_l[slot * C::RPB + row_a] = L_a;
                a.ws_l[slot * C::RPB + row_b] = L_b;
            }
        }

        if (warp == 1 && last) HOGATT_TL(1, 900);
        // ---- hand the stage back to the producer ----
        if (wrote_scratch || nvalid < C::TILE) fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(empty0 + 8 * stage);

        if (++j == TH) {
            j = 0;
            ++u;
        }
    }
    if constexpr (CL) {
        constexpr int CTHREADS = C::NCW * 32;
        if (!waited) {                   // a CTA without tiles
            pdl_wait();
            pdl_trigger();
        }
        if (rq_by_consumers && it == 0)  // a CTA without tiles still writes its share of the rotated queries
            write_rotated_queries<T>(a.q, a.rq, a.cos, a.sin, a.F, a.W, a.Hq, a.S, HD, a.R,
                                     blockIdx.x * CTHREADS + tid - 32, gridDim.x * CTHREADS);
        // ---- leave this warp's private result in shared memory ----
        l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
        l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
        l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
        l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
        if (it == 0) {                   // the accumulators were never initialised
            m_a = m_b = -INFINITY;
            l_a = l_b = 0.f;
#pragma unroll
            for (int n = 0; n < C::NT_O; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
        }
        float* const scr = reinterpret_cast<float*>(stages);
        named_barrier_sync(1, CTHREADS);                  // every consumer warp is done with the K/V stages
        {
            float* part = scr + (size_t)cw * C::CL_PART_FLOATS;
#pragma unroll
            for (int n = 0; n < C::NT_O; ++n) {
                *reinterpret_cast<float2*>(part + quad * C::OPITCH + n * 8 + qlane * 2) = make_float2(o[n][0], o[n][1]);
                *reinterpret_cast<float2*>(part + (quad + 8) * C::OPITCH + n * 8 + qlane * 2) = make_float2(o[n][2], o[n][3]);
            }
            if (qlane == 0) {
                scr[C::CL_STAT + cw * 16 + quad] = m_a;
                scr[C::CL_STAT + cw * 16 + quad + 8] = m_b;
                scr[C::CL_STAT + C::NCW * 16 + cw * 16 + quad] = l_a;
                scr[C::CL_STAT + C::NCW * 16 + cw * 16 + quad + 8] = l_b;
            }
        }
        cluster_sync_all();
        if (warp == 1) HOGATT_TL(1, 901);

        // ---- merge rows crank, crank + CS, ... of the block over every warp of every CTA ----
        const int P = CS * C::NSLICE;                     // partials per row (<= 128)
        const int RC = (C::RPB - crank + CS - 1) / CS;    // rows this CTA finishes (CS <= 16 <= RPB: at least one)
        const int SPLIT = max(1, C::NCW / ((C::RPB + CS - 1) / CS));   // warps sharing one row, each takes partials p % SPLIT == sub
        const int ntask = RC * SPLIT;
        const uint32_t scr_addr = smem_u32(scr);
        for (int task = cw; task < ntask; task += C::NCW) {
            const int ri = task / SPLIT, sub = task % SPLIT;
            const int r = crank + ri * CS;
            const int mt_r = r >> 4, rr = r & 15;
            float mp[4], lp[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int p = lane + 32 * k;
                mp[k] = -INFINITY;
                lp[k] = 0.f;
                if (p < P) {
                    const int wp = (p % C::NSLICE) * MT + mt_r;
                    const uint32_t ad = map_to_cta(scr_addr + (C::CL_STAT + wp * 16 + rr) * 4, p / C::NSLICE);
                    mp[k] = ld_cluster_f(ad);
                    lp[k] = ld_cluster_f(ad + C::NCW * 16 * 4);
                }
            }
            float M = fmaxf(fmaxf(mp[0], mp[1]), fmaxf(mp[2], mp[3]));
#pragma unroll
            for (int sh = 16; sh > 0; sh >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, sh));
            const float mu = (M == -INFINITY) ? 0.f : M;
            const float w0 = exp2f(mp[0] - mu), w1 = exp2f(mp[1] - mu), w2 = exp2f(mp[2] - mu), w3 = exp2f(mp[3] - mu);
            float den = lp[0] * w0 + lp[1] * w1 + lp[2] * w2 + lp[3] * w3;
#pragma unroll
            for (int sh = 16; sh > 0; sh >>= 1) den += __shfl_xor_sync(0xffffffffu, den, sh);
            const bool act = lane * 4 < HD;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            constexpr int UNR = 8;
            for (int p0 = sub; p0 < P; p0 += SPLIT * UNR) {
                float4 x[UNR];
#pragma unroll
                for (int i = 0; i < UNR; ++i) {
                    const int p = p0 + i * SPLIT;
                    x[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (p < P && act) {
                        const int wp = (p % C::NSLICE) * MT + mt_r;
                        x[i] = ld_cluster_f4(map_to_cta(
                            scr_addr + (wp * C::CL_PART_FLOATS + rr * C::OPITCH + lane * 4) * 4, p / C::NSLICE));
                    }
                }
#pragma unroll
                for (int i = 0; i < UNR; ++i) {
                    const int p = p0 + i * SPLIT;
                    const int hi = (p >> 5) & 3;
                    const float wgt = __shfl_sync(0xffffffffu, hi == 0 ? w0 : (hi == 1 ? w1 : (hi == 2 ? w2 : w3)), p & 31);
                    acc.x = fmaf(x[i].x, wgt, acc.x);
                    acc.y = fmaf(x[i].y, wgt, acc.y);
                    acc.z = fmaf(x[i].z, wgt, acc.z);
                    acc.w = fmaf(x[i].w, wgt, acc.w);
                }
            }
            if (act) *reinterpret_cast<float4*>(scr + C::CL_ACC + task * HD + lane * 4) = acc;
            if (lane == 0) scr[C::CL_DEN + task] = den;
        }
        named_barrier_sync(1, CTHREADS);
        {
            const int unit = (int)(blockIdx.x / CS);
            const int rb_u = unit / a.Hkv, hkv_u = unit % a.Hkv;
            const OutputTargets<T> dst(a);
            for (int item = tid - 32; item < RC * (HD / 4); item += CTHREADS) {
                const int ri = item / (HD / 4), c4 = item % (HD / 4);
                const int gr = rb_u * C::RPB + crank + ri * CS;
                if (gr >= a.rows_total) continue;
                float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int sub = 0; sub < SPLIT; ++sub) {
                    const float4 y = *reinterpret_cast<const float4*>(scr + C::CL_ACC + (ri * SPLIT + sub) * HD + c4 * 4);
                    sum.x += y.x;
                    sum.y += y.y;
                    sum.z += y.z;
                    sum.w += y.w;
                }
                const float den = scr[C::CL_DEN + ri * SPLIT];
                const float inv = den > 0.f ? 1.f / den : 0.f;
                if (!(den > 0.f)) sum = make_float4(0.f, 0.f, 0.f, 0.f);
                const RowId id = decode_row(gr, a.G, a.S);
                const size_t offset = dst.row_offset(id.w, hkv_u * a.G + id.g, id.s, a.S, HD) + c4 * 4;
                uint2 packed;
                packed.x = pack2<T>(sum.x * inv, sum.y * inv);
                packed.y = pack2<T>(sum.z * inv, sum.w * inv);
                for (int b = 0; b < dst.nbases; ++b) *reinterpret_cast<uint2*>(dst.base(b) + offset) = packed;
            }
        }
        if (warp == 1) HOGATT_TL(1, 902);
        cluster_sync_all();              // no CTA leaves while another may still read its shared memory
    }
    if (tid == 32) HOGATT_TRACE(a.debug_id, 3);
#ifdef HOGATT_TIMELINE
    if (warp == 1 && lane == 0) {
        atomicMax(&g_span[1], global_timer_ns_());
        g_cta_t[2][blockIdx.x] = global_timer_ns_();
    }
#endif
}

}  // namespace hogatt
