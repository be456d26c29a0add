// C ABI of libhogatt_b200.so (declared in include/hogatt.h): argument validation, kernel choice,
// workspace carving and launches.  No allocation, no synchronisation, and no static device buffers, with one
// declared exception: the fixed scratch array that hogatt_fused_launch_static uses in place of a workspace.
#include <algorithm>
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "hogatt_device.cuh"
#include "hogatt_fma.cuh"
#include "hogatt_merge.cuh"
#include "hogatt_mma.cuh"
#include "hogatt_paged.cuh"
#include "hogatt_cache.cuh"
#include "hogatt_dense.cuh"

#include <mutex>
#include <unordered_map>

namespace hogatt {
namespace {

thread_local int tl_last_cuda_error = 0;

#define HOGATT_CUDA_OK(expr)                         \
    do {                                             \
        cudaError_t err__ = (expr);                  \
        if (err__ != cudaSuccess) {                  \
            tl_last_cuda_error = (int)err__;         \
            (void)cudaGetLastError();                \
            return HOGATT_ERR_CUDA;                  \
        }                                            \
    } while (0)

constexpr int kMaxDevices = 64;

struct DeviceInfo {
    std::atomic<int> sms{0};
    std::atomic<int> smem_optin{0};
};
DeviceInfo g_devices[kMaxDevices];

int current_device_info(int* dev, int* sms, int* smem_optin) {
    HOGATT_CUDA_OK(cudaGetDevice(dev));
    if (*dev < 0 || *dev >= kMaxDevices) return HOGATT_ERR_CUDA;
    DeviceInfo& d = g_devices[*dev];
    int n = d.sms.load(std::memory_order_acquire);
    if (n == 0) {
        int s = 0, m = 0;
        HOGATT_CUDA_OK(cudaDeviceGetAttribute(&s, cudaDevAttrMultiProcessorCount, *dev));
        HOGATT_CUDA_OK(cudaDeviceGetAttribute(&m, cudaDevAttrMaxSharedMemoryPerBlockOptin, *dev));
        if (const char* ms = getenv("HOGATT_WAIT_LIMIT_MS")) {      // tests of the give-up path shorten every bounded wait
            const unsigned long long ns = (unsigned long long)std::max(1, atoi(ms)) * 1000000ull;
            HOGATT_CUDA_OK(cudaMemcpyToSymbol(g_wait_limit_ns, &ns, sizeof(ns)));
        }
        d.smem_optin.store(m, std::memory_order_release);
        d.sms.store(s, std::memory_order_release);
        n = s;
    }
    *sms = n;
    *smem_optin = d.smem_optin.load(std::memory_order_acquire);
    return HOGATT_OK;
}

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) once per (kernel instantiation, device).
template <class Kernel>
int ensure_smem_limit(Kernel kernel, int dev, size_t bytes, std::atomic<size_t>* granted /*[kMaxDevices]*/) {
    if (bytes <= 48 * 1024) return HOGATT_OK;
    if (granted[dev].load(std::memory_order_acquire) >= bytes) return HOGATT_OK;
    HOGATT_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
    granted[dev].store(bytes, std::memory_order_release);
    return HOGATT_OK;
}

// Launch with the programmatic-stream-serialization attribute: the kernel may be scheduled while its
// stream predecessor is still running (each of our kernels calls griddepcontrol.wait before it touches
// global memory that earlier work may write -- everything except the K/V rows of fragments the caller
// declared stable).  On unless HOGATT_PDL=0 is set in the environment when the library is first used.
bool pdl_enabled() {
    static const bool on = [] {
        const char* v = getenv("HOGATT_PDL");
        return !(v && v[0] == '0');
    }();
    return on;
}

// HOGATT_DENSE=0 in the environment keeps AUTO away from the tcgen05 kernel (A/B measurements).
bool dense_disabled() {
    static const bool off = [] {
        const char* v = getenv("HOGATT_DENSE");
        return v && v[0] == '0';
    }();
    return off;
}

// HOGATT_HOST_PLAN=0 in the environment (read when the library is first used) makes every call derive its
// tiles on the device even when the caller gave host_lengths: for A/B measurements.
bool host_plan_disabled() {
    static const bool off = [] {
        const char* v = getenv("HOGATT_HOST_PLAN");
        return v && v[0] == '0';
    }();
    return off;
}

template <class... KArgs, class... Args>
cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

size_t dtype_size(int dtype) { return dtype == HOGATT_F32 ? 4 : 2; }

// What will run for this problem.
struct Resolved {
    int kernel;          // HOGATT_KERNEL_FMA or HOGATT_KERNEL_MMA
    int mt;              // m-tiles per CTA (tensor-core kernel)
    int rows_per_block;
    int tile_tokens;
    int row_blocks;
    int units;
    int cluster_mode;    // -1 never (HOGATT_KERNEL_MMA), 0 let choose_cluster decide (AUTO), 1 required (HOGATT_KERNEL_MMA_CLUSTER)
    int cluster;         // CTAs per cluster of the self-merging variant, 0 = persistent grid + merge kernel
    bool cluster_forced;
};

bool mma_eligible(const hogatt_problem* p) {
    if (p->dtype != HOGATT_F16 && p->dtype != HOGATT_BF16) return false;
    if (p->E != p->Ev || (p->E != 64 && p->E != 128)) return false;
    return true;
}

// The tcgen05 kernel: 16-bit types, head size 128, at least one full 128-row query block per kv head, and a block
// must be a whole box of the rotated-query tensor [F, W, Hkv, G*S, E]: either whole workers (G*S divides 128) or a
// slice of one worker's rows (128 divides G*S).  Tensor maps travel in the kernel arguments, hence the fragment cap.
bool dense_eligible(const hogatt_problem* p) {
    if (p->dtype != HOGATT_F16 && p->dtype != HOGATT_BF16) return false;
    if (p->E != 128 || p->Ev != 128 || p->F > kDenseMaxFragments) return false;
    const int64_t gs = (int64_t)(p->Hq / p->Hkv) * p->S;
    if ((int64_t)p->W * gs < kDenseRows) return false;
    return gs <= kDenseRows ? kDenseRows % gs == 0 : gs % kDenseRows == 0;
}

bool fma_eligible(const hogatt_problem* p) {
    const int vec = 16 / (int)dtype_size(p->dtype);
    if (p->Ev != 32 && p->Ev != 64 && p->Ev != 128 && p->Ev != 256) return false;
    if (p->E < vec || p->E > 256 || p->E % vec != 0) return false;
    return true;
}

int resolve(const hogatt_problem* p, Resolved* r) {
    if (p == nullptr) return HOGATT_ERR_NULL_POINTER;
    if (p->F <= 0 || p->W <= 0 || p->Hq <= 0 || p->Hkv <= 0 || p->E <= 0 || p->Ev <= 0 || p->S <= 0)
        return HOGATT_ERR_BAD_SHAPE;
    if (p->Hq % p->Hkv != 0) return HOGATT_ERR_BAD_SHAPE;
    if (p->F > HOGATT_MAX_FRAGMENTS) return HOGATT_ERR_TOO_MANY_FRAGMENTS;
    if (p->dtype != HOGATT_F32 && p->dtype != HOGATT_F16 && p->dtype != HOGATT_BF16) return HOGATT_ERR_UNSUPPORTED_DTYPE;
    const int64_t rows_total = (int64_t)p->W * (p->Hq / p->Hkv) * p->S;
    if (rows_total > (1 << 24) || (int64_t)p->F * p->W * p->S > (1 << 26)) return HOGATT_ERR_TOO_LARGE;
    // the rotated-query side output [F,W,Hq,S,E] is indexed with 32-bit element counts in the kernels
    if ((int64_t)p->F * p->W * p->Hq * p->S * std::max(p->E, 8) >= ((int64_t)1 << 31)) return HOGATT_ERR_TOO_LARGE;
    int kernel = p->kernel;
    r->cluster_mode = kernel == HOGATT_KERNEL_MMA ? -1 : (kernel == HOGATT_KERNEL_MMA_CLUSTER ? 1 : 0);
    r->cluster = 0;
    r->cluster_forced = kernel == HOGATT_KERNEL_MMA_CLUSTER;
    if (kernel == HOGATT_KERNEL_MMA_CLUSTER) kernel = HOGATT_KERNEL_MMA;
    if (kernel == HOGATT_KERNEL_AUTO)
        kernel = (dense_eligible(p) && !dense_disabled()) ? HOGATT_KERNEL_DENSE
                                                           : (mma_eligible(p) ? HOGATT_KERNEL_MMA : HOGATT_KERNEL_FMA);
    if (kernel == HOGATT_KERNEL_DENSE) {
        if (!dense_eligible(p)) return HOGATT_ERR_BAD_KERNEL_CHOICE;
        r->cluster_mode = -1;
        r->mt = 0;
        r->rows_per_block = kDenseRows;
        r->tile_tokens = kDenseTile;
    } else if (kernel == HOGATT_KERNEL_MMA) {
        if (!mma_eligible(p)) return HOGATT_ERR_BAD_KERNEL_CHOICE;
        r->mt = rows_total <= 16 ? 1 : (rows_total <= 32 ? 2 : 4);
        r->rows_per_block = 16 * r->mt;
        r->tile_tokens = p->E == 128 ? 128 : 256;
    } else if (kernel == HOGATT_KERNEL_FMA) {
        if (!fma_eligible(p)) return HOGATT_ERR_UNSUPPORTED_HEAD_DIM;
        r->mt = 1;
        r->rows_per_block = kFmaRows;
        r->tile_tokens = kFmaTile;
    } else {
        return HOGATT_ERR_BAD_KERNEL_CHOICE;
    }
    r->kernel = kernel;
    r->row_blocks = (int)((rows_total + r->rows_per_block - 1) / r->rows_per_block);
    const int64_t units = (int64_t)r->row_blocks * p->Hkv;
    if (units > (1 << 24)) return HOGATT_ERR_TOO_LARGE;
    r->units = (int)units;
    return HOGATT_OK;
}

struct WorkspaceLayout {
    size_t header, o, m, l, rq, total;
    int parts;
};

WorkspaceLayout carve(const hogatt_problem* p, const Resolved& r, int grid) {
    WorkspaceLayout w;
    w.parts = max_parts_per_unit(r.units, grid);
    const size_t slots = (size_t)r.units * w.parts * r.rows_per_block;
    w.header = 0;
    w.o = 256;
    w.m = w.o + align_up(slots * p->Ev * sizeof(float), 256);
    w.l = w.m + align_up(slots * sizeof(float), 256);
    w.rq = w.l + align_up(slots * sizeof(float), 256);
    // the tcgen05 kernel reads rotated queries from memory: room for them in case the caller does not want them back
    w.total = w.rq + (r.kernel == HOGATT_KERNEL_DENSE
                          ? align_up((size_t)p->F * p->W * p->Hq * p->S * p->E * dtype_size(p->dtype), 256) : 0);
    return w;
}

// Largest cluster the self-merging variant could use if every cluster size up to 16 were available:
// host-only bound, for hogatt_plan_describe.
int cluster_upper_bound(const Resolved& r, int sms) {
    if (r.kernel != HOGATT_KERNEL_MMA || r.cluster_mode < 0) return 0;
    const int cs = std::min(16, sms / std::max(r.units, 1));
    return cs >= 2 ? cs : 0;
}

int64_t tiles_upper_bound(const hogatt_problem* p, const Resolved& r) {
    int64_t th = 0;
    for (int f = 0; f < p->F; ++f) {
        int rows = p->fragment_rows[f] < 0 ? 0 : p->fragment_rows[f];
        if (p->host_lengths) rows = std::max(0, std::min(rows, p->host_lengths[f]));
        th += ceil_div(rows, r.tile_tokens);
    }
    return th;
}

// How many query rows a CTA of the mma.sync kernel keeps (16, 32 or 64): resolve() takes the smallest block that
// holds all W*G*S rows of a kv head, so that every key is fetched once.  With few kv heads and a short context that
// leaves each CTA one or two tiles behind a start-up that grows with the block (query rows to rotate and stage,
// warps to fold, partials per row to merge), and smaller blocks -- more units, every key fetched once per row block,
// the repeats served by L2 since the row blocks of a head walk the keys together -- are faster.  Fitted on B200
// (microseconds per call, n = tiles per CTA): 16 rows 9.0 + 1.03 n, 32 rows 13.4 + 1.27 n, 64 rows 18.5 + 2.64 n;
// e.g. 64 rows over 2 kv heads and 16 K keys: 23.1 us as one 64-row block (n = 1.7), 17.8 as two of 32, 16.1 as
// four of 16 (n = 6.9); 20 rows over 8 kv heads stay one 32-row block (22.2 against 23.2 us).
void refine_row_blocks(const hogatt_problem* p, Resolved* r, int grid, int64_t tiles_per_unit) {
    if (r->kernel != HOGATT_KERNEL_MMA || r->cluster_forced || r->mt <= 1 || tiles_per_unit <= 0 || grid <= 0) return;
    static const float kFixed[3] = {9.0f, 13.4f, 18.5f}, kPerTile[3] = {1.03f, 1.27f, 2.64f};
    const int64_t rows_total = (int64_t)p->W * (p->Hq / p->Hkv) * p->S;
    // (fitted on calls of a few tiles per CTA and only applied there: with many tiles per CTA the largest block,
    // which fetches every key once, stays)
    if ((int64_t)r->units * tiles_per_unit >= (int64_t)8 * grid) return;
    int best = r->mt;
    float best_t = 0.f;
    for (int i = 0, mt = 1; mt <= r->mt; ++i, mt *= 2) {
        const int64_t blocks = (rows_total + 16 * mt - 1) / (16 * mt);
        const float t = kFixed[i] + kPerTile[i] * (float)(blocks * p->Hkv * tiles_per_unit) / (float)grid;
        if (mt == 1 || t < best_t) {
            best = mt;
            best_t = t;
        }
    }
    if (best == r->mt) return;
    r->mt = best;
    r->rows_per_block = 16 * best;
    r->row_blocks = (int)((rows_total + r->rows_per_block - 1) / r->rows_per_block);
    r->units = r->row_blocks * p->Hkv;
}

int grid_size(const hogatt_problem* p, int sms) {
    int grid = sms;
    if (p->max_ctas > 0 && p->max_ctas < grid) grid = p->max_ctas;
    return grid;
}

// ---- launch helpers, one per kernel family ------------------------------------------------------

// Upper limit on CTAs per cluster: 16 (the hardware's), or HOGATT_MAX_CLUSTER from the environment
// (2..16, read when the library is first used; for experiments with the cluster shape).
int max_cluster_size() {
    static const int cap = [] {
        const char* v = getenv("HOGATT_MAX_CLUSTER");
        const int n = v ? atoi(v) : 16;
        return n < 2 ? 2 : (n > 16 ? 16 : n);
    }();
    return cap;
}

// How many clusters of `cs` CTAs of the cluster variant the device holds at once (0 on failure), asked
// once per (kernel instantiation, device, size).  It depends on how the SMs are grouped on the part: a
// B200 with one ~200 KB CTA per SM holds 74 clusters of 2, 33 of 4, 15 of 8 or 9, 11 of 10, 7 of 11..16.
template <class T, int HD, int MT>
std::atomic<size_t>* cluster_smem_granted() {
    static std::atomic<size_t> granted[kMaxDevices];
    return granted;
}

template <class T, int HD, int MT>
int mma_resident_clusters(int dev, size_t smem, int cs) {
    std::atomic<size_t>* granted = cluster_smem_granted<T, HD, MT>();
    static std::atomic<int> wide_ok[kMaxDevices];                      // clusters of more than 8 CTAs are opt-in
    static std::atomic<int> resident[kMaxDevices][17];                 // +1; 0 = not asked yet
    using C = MmaCfg<HD, MT>;
    auto kernel = mma_attention_kernel<T, HD, MT, true>;
    int have = resident[dev][cs].load(std::memory_order_acquire);
    if (have) return have - 1;
    if (ensure_smem_limit(kernel, dev, smem, granted) != HOGATT_OK) return 0;
    if (!wide_ok[dev].load(std::memory_order_acquire)) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) return 0;
        wide_ok[dev].store(1, std::memory_order_release);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(cs);
    cfg.blockDim = dim3(C::THREADS);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)cs;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess) {
        cudaGetLastError();
        n = 0;
    }
    resident[dev][cs].store(n + 1, std::memory_order_release);
    return n;
}

// The largest cluster size (2..16) at which one cluster per unit is resident all at once; 0 if none.
template <class T, int HD, int MT>
int mma_best_cluster(int dev, int F, int smem_optin, int units, int sms) {
    const size_t smem = mma_smem_bytes<HD, MT>(F);
    if (smem > (size_t)smem_optin) return 0;
    for (int cs = std::min(max_cluster_size(), sms / std::max(units, 1)); cs >= 2; --cs)
        if (mma_resident_clusters<T, HD, MT>(dev, smem, cs) >= units) return cs;
    return 0;
}

template <class T>
int mma_best_cluster_dims(int HD, int MT, int dev, int F, int smem_optin, int units, int sms) {
    if (HD == 128) {
        if (MT == 1) return mma_best_cluster<T, 128, 1>(dev, F, smem_optin, units, sms);
        if (MT == 2) return mma_best_cluster<T, 128, 2>(dev, F, smem_optin, units, sms);
        return mma_best_cluster<T, 128, 4>(dev, F, smem_optin, units, sms);
    }
    if (MT == 1) return mma_best_cluster<T, 64, 1>(dev, F, smem_optin, units, sms);
    if (MT == 2) return mma_best_cluster<T, 64, 2>(dev, F, smem_optin, units, sms);
    return mma_best_cluster<T, 64, 4>(dev, F, smem_optin, units, sms);
}

// CTAs per cluster if this problem runs as the self-merging cluster variant on the current device, else 0
// (persistent grid + merge kernel).  The cluster variant saves the partials' trip through the workspace and the
// second launch, but it only uses units * cluster SMs (at most 16 per unit, and only as many clusters as are resident
// at once), and one SM pulls about 66 GB/s.  Measured on B200 it loses to the persistent grid everywhere since the
// merge step handles many partials per row in one round trip (one rank's share of an 8-way kv-head split: 16,384
// keys 8.9 us against 14.8, 139,264 keys 20.7 us against 79), so AUTO never takes it; it runs on request only
// (HOGATT_KERNEL_MMA_CLUSTER).
int choose_cluster(const hogatt_problem* p, const Resolved& r, int dev, int sms, int smem_optin, int64_t tiles_per_unit) {
    (void)tiles_per_unit;
    if (r.kernel != HOGATT_KERNEL_MMA || r.cluster_mode <= 0 || 2 * r.units > sms) return 0;
    int cs = 0;
    if (p->dtype == HOGATT_F16) cs = mma_best_cluster_dims<__half>(p->E, r.mt, dev, p->F, smem_optin, r.units, sms);
    if (p->dtype == HOGATT_BF16) cs = mma_best_cluster_dims<__nv_bfloat16>(p->E, r.mt, dev, p->F, smem_optin, r.units, sms);
    return cs;
}

// cluster == 0: persistent grid of `grid` CTAs (merge_kernel must follow).
// cluster >= 2: units * cluster CTAs in clusters of `cluster`; the kernel merges by itself.
template <class T, int HD, int MT>
int launch_mma(const KernelArgs& args, int F, int dev, int smem_optin, int grid, int cluster, bool evict_first,
               cudaStream_t stream, int extra_flags = 0) {
    using C = MmaCfg<HD, MT>;
    const size_t smem = mma_smem_bytes<HD, MT>(F);
    if (smem > (size_t)smem_optin) return HOGATT_ERR_TOO_MANY_FRAGMENTS;
    if (cluster == 0) {
        static std::atomic<size_t> granted[kMaxDevices];
        int rc = ensure_smem_limit(mma_attention_kernel<T, HD, MT, false>, dev, smem, granted);
        if (rc != HOGATT_OK) return rc;
        HOGATT_CUDA_OK(launch_kernel(mma_attention_kernel<T, HD, MT, false>, dim3(grid), dim3(C::THREADS), smem, stream,
                                     args, (evict_first ? 1 : 0) | extra_flags));
        return HOGATT_OK;
    }
    // the wide-cluster opt-in was set when choose_cluster() asked for the residency; the shared-memory limit
    // too, but for the fragment count of that call
    int rc = ensure_smem_limit(mma_attention_kernel<T, HD, MT, true>, dev, smem, cluster_smem_granted<T, HD, MT>());
    if (rc != HOGATT_OK) return rc;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(C::THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)cluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    HOGATT_CUDA_OK(cudaLaunchKernelEx(&cfg, mma_attention_kernel<T, HD, MT, true>, args, (int)((evict_first ? 1 : 0) | extra_flags)));
    return HOGATT_OK;
}

template <class T>
int launch_mma_dims(const KernelArgs& args, int F, int HD, int MT, int dev, int smem_optin, int grid, int cluster, bool ef,
                    cudaStream_t stream, int extra_flags = 0) {
    if (HD == 128) {
        if (MT == 1) return launch_mma<T, 128, 1>(args, F, dev, smem_optin, grid, cluster, ef, stream, extra_flags);
        if (MT == 2) return launch_mma<T, 128, 2>(args, F, dev, smem_optin, grid, cluster, ef, stream, extra_flags);
        return launch_mma<T, 128, 4>(args, F, dev, smem_optin, grid, cluster, ef, stream, extra_flags);
    }
    if (MT == 1) return launch_mma<T, 64, 1>(args, F, dev, smem_optin, grid, cluster, ef, stream, extra_flags);
    if (MT == 2) return launch_mma<T, 64, 2>(args, F, dev, smem_optin, grid, cluster, ef, stream, extra_flags);
    return launch_mma<T, 64, 4>(args, F, dev, smem_optin, grid, cluster, ef, stream, extra_flags);
}

template <class T, int EV>
int launch_fma(const KernelArgs& args, int dev, int smem_optin, int grid, cudaStream_t stream) {
    static std::atomic<size_t> granted[kMaxDevices];
    const size_t smem = fma_smem_bytes(args.E, EV, args.F);
    if (smem > (size_t)smem_optin) return HOGATT_ERR_UNSUPPORTED_HEAD_DIM;
    int rc = ensure_smem_limit(fma_attention_kernel<T, EV>, dev, smem, granted);
    if (rc != HOGATT_OK) return rc;
    HOGATT_CUDA_OK(launch_kernel(fma_attention_kernel<T, EV>, dim3(grid), dim3(kFmaThreads), smem, stream, args));
    return HOGATT_OK;
}

template <class T>
int launch_fma_dims(const KernelArgs& args, int dev, int smem_optin, int grid, cudaStream_t stream) {
    switch (args.Ev) {
        case 32: return launch_fma<T, 32>(args, dev, smem_optin, grid, stream);
        case 64: return launch_fma<T, 64>(args, dev, smem_optin, grid, stream);
        case 128: return launch_fma<T, 128>(args, dev, smem_optin, grid, stream);
        case 256: return launch_fma<T, 256>(args, dev, smem_optin, grid, stream);
    }
    return HOGATT_ERR_UNSUPPORTED_HEAD_DIM;
}

// The merge step after a persistent-grid attention kernel.  Up to 32 partial slots per unit: one warp per output row
// (lean instantiation; 8 kv heads on one GPU leave 19-20 partials per row).  More -- kv heads sharded over GPUs, one
// unit cut into 37 ... 148 partials -- one CTA per row whose eight warps share the partials (one memory round trip
// instead of one per 24 partials), as long as that grid stays small; otherwise the batched one-warp-per-row kernel.
template <class T>
int launch_merge(const KernelArgs& args, const Resolved& r, cudaStream_t stream) {
    // Partials a row can have: what the workspace reserves per unit, or -- under a host plan, where the CTA count is
    // known here -- what the ranges can actually leave (exactly ctas / units when that divides: aligned ranges).
    int bound = args.parts_per_unit;
    if (args.host_plan && r.units > 0)
        bound = std::min(bound, ceil_div(args.plan_ctas, r.units) + (args.plan_ctas % r.units == 0 ? 0 : 1));
    if (bound > 32 && (int64_t)r.units * r.rows_per_block <= 4096) {
        dim3 wgrid((unsigned)r.units, (unsigned)r.rows_per_block);
        // One CTA per row.  Up to 64 partials: four warps x 16 partials under 102 registers, a CTA that fits on an SM
        // beside a resident attention CTA (0.04-0.2 us per call over the next one); up to 96: four warps x 24 (168
        // registers); 128-148 (one kv head per GPU): eight warps x 24 -- four warps would take two round trips there
        // (8.7 -> 9.3 us per call).  (Two round trips of 32 on the one-warp-per-row kernel instead, for 33-64 partials:
        // 12.2 us against 9.6.)
        if (bound <= 4 * 16)
            HOGATT_CUDA_OK(launch_kernel(merge_wide_kernel<T, 4, 16>, wgrid, dim3(4 * 32), 0, stream, args));
        else if (bound <= 4 * 24)
            HOGATT_CUDA_OK(launch_kernel(merge_wide_kernel<T, 4>, wgrid, dim3(4 * 32), 0, stream, args));
        else
            HOGATT_CUDA_OK(launch_kernel(merge_wide_kernel<T>, wgrid, dim3(kWideWarps * 32), 0, stream, args));
        return HOGATT_OK;
    }
    dim3 mgrid((unsigned)r.units, (unsigned)ceil_div(r.rows_per_block, kMergeWarps));
    if (args.parts_per_unit <= 4)           // units of many query rows, cut into few partials each: lean instantiations
        HOGATT_CUDA_OK(launch_kernel(merge_kernel<T, 1, 4>, mgrid, dim3(kMergeWarps * 32), 0, stream, args));
    else if (args.parts_per_unit <= 8)
        HOGATT_CUDA_OK(launch_kernel(merge_kernel<T, 1, 8>, mgrid, dim3(kMergeWarps * 32), 0, stream, args));
    else if (bound <= 32) {
        // One warp per row, two warps per CTA: 64 threads x 150-190 registers fit on an SM BESIDE a resident attention
        // CTA (192 threads x 255 registers leave 16 K registers), four warps do not.  With programmatic dependent
        // launch that decides whether this grid is already resident when the attention grid drains, and whether the
        // next call's attention CTAs can start on the SMs this grid occupies (measured: 18.8 -> 17.2 us per call at
        // 16 K keys, 24.2 -> 22.2 at GQA 5).  The first round trip fetches 16, 24 or 32 partials per row; the fewer
        // loads a warp issues the sooner they are back (16 instead of 24 at 16 partials per row: -0.3 us per call).
        dim3 g2((unsigned)r.units, (unsigned)ceil_div(r.rows_per_block, 2));
        if (bound <= 16)
            HOGATT_CUDA_OK(launch_kernel(merge_kernel<T, 1, 16, 2>, g2, dim3(64), 0, stream, args));
        else if (bound <= 24)
            HOGATT_CUDA_OK(launch_kernel(merge_kernel<T, 1, 24, 2>, g2, dim3(64), 0, stream, args));
        else
            HOGATT_CUDA_OK(launch_kernel(merge_kernel<T, 1, 32, 2>, g2, dim3(64), 0, stream, args));
    }
    else
        HOGATT_CUDA_OK(launch_kernel(merge_kernel<T, 5>, mgrid, dim3(kMergeWarps * 32), 0, stream, args));
    return HOGATT_OK;
}

// ---- tcgen05 kernel: tensor maps and launch ------------------------------------------------------------------
// cuTensorMapEncodeTiled comes from the driver; it is looked up through the runtime so that the library links
// against nothing but cudart.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn tensor_map_encoder() {
    static EncodeTiledFn fn = [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess) {
            (void)cudaGetLastError();
            ptr = nullptr;
        }
        return reinterpret_cast<EncodeTiledFn>(ptr);
    }();
    return fn;
}

// A tiled map with the 128-byte swizzle over a dense row-major tensor of 16-bit elements: dims[0] is the contiguous
// one, box[0] = 64 elements = 128 bytes.
int encode_map(CUtensorMap* out, const void* base, int dtype, int rank, const cuuint64_t* dims, const cuuint32_t* box) {
    EncodeTiledFn fn = tensor_map_encoder();
    if (!fn) return HOGATT_ERR_CUDA;
    cuuint64_t strides[4];
    cuuint64_t acc = 2;
    for (int i = 0; i + 1 < rank; ++i) {
        acc *= dims[i];
        strides[i] = acc;
    }
    const cuuint32_t ones[5] = {1, 1, 1, 1, 1};
    const CUresult rc = fn(out, dtype == HOGATT_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                           (cuuint32_t)rank, const_cast<void*>(base), dims, strides, box, ones, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) {
        tl_last_cuda_error = (int)rc;
        return HOGATT_ERR_CUDA;
    }
    return HOGATT_OK;
}

// Fragment maps are cached by (pointer, rows, heads, dtype): preallocated slabs keep their pointers for the whole
// generation, so a decode step encodes nothing.
struct MapKey {
    const void* ptr;
    int rows, hkv, dtype;
    bool operator==(const MapKey& o) const { return ptr == o.ptr && rows == o.rows && hkv == o.hkv && dtype == o.dtype; }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        return std::hash<const void*>()(k.ptr) ^ ((size_t)k.rows * 0x9E3779B97F4A7C15ull) ^ ((size_t)k.hkv << 48) ^ ((size_t)k.dtype << 56);
    }
};
int fragment_map(const void* ptr, int rows, int Hkv, int dtype, CUtensorMap* out) {
    static std::mutex mu;
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    const MapKey key{ptr, rows, Hkv, dtype};
    {
        std::lock_guard<std::mutex> lock(mu);
        auto it = cache.find(key);
        if (it != cache.end()) {
            *out = it->second;
            return HOGATT_OK;
        }
    }
    const cuuint64_t dims[3] = {128, (cuuint64_t)rows, (cuuint64_t)Hkv};
    const cuuint32_t box[3] = {64, kDenseTile, 1};
    const int rc = encode_map(out, ptr, dtype, 3, dims, box);
    if (rc != HOGATT_OK) return rc;
    std::lock_guard<std::mutex> lock(mu);
    if (cache.size() >= 8192) cache.clear();
    cache.emplace(key, *out);
    return HOGATT_OK;
}

template <class T>
int launch_dense(const KernelArgs& args, const void* q_rot, int dtype, int dev, int smem_optin, int grid, cudaStream_t stream) {
    static std::atomic<size_t> granted[kMaxDevices];
    const size_t smem = dense_smem_bytes(args.F);
    if (smem > (size_t)smem_optin) return HOGATT_ERR_TOO_MANY_FRAGMENTS;
    int rc = ensure_smem_limit(dense_attention_kernel<T>, dev, smem, granted);
    if (rc != HOGATT_OK) return rc;
    DenseMaps maps;
    memset(&maps, 0, sizeof(maps));
    for (int f = 0; f < args.F; ++f) {
        if (args.ft.e[f].rows == 0) continue;             // never addressed: no tile lies in an empty fragment
        rc = fragment_map(args.ft.e[f].k, args.ft.e[f].rows, args.Hkv, dtype, &maps.k[f]);
        if (rc == HOGATT_OK) rc = fragment_map(args.ft.e[f].v, args.ft.e[f].rows, args.Hkv, dtype, &maps.v[f]);
        if (rc != HOGATT_OK) return rc;
    }
    {   // rotated queries [F, W, Hq, S, E] seen as [F, W, Hkv, G*S, E]; a 128-row block is one box
        const int gs = args.G * args.S;
        const cuuint64_t dims[5] = {128, (cuuint64_t)gs, (cuuint64_t)args.Hkv, (cuuint64_t)args.W, (cuuint64_t)args.F};
        const cuuint32_t box[5] = {64, (cuuint32_t)std::min(gs, kDenseRows), 1, (cuuint32_t)(gs < kDenseRows ? kDenseRows / gs : 1), 1};
        rc = encode_map(&maps.q, q_rot, dtype, 5, dims, box);
        if (rc != HOGATT_OK) return rc;
    }
    dense_attention_kernel<T><<<dim3(grid), dim3(kDenseThreads), smem, stream>>>(args, maps);
    HOGATT_CUDA_OK(cudaGetLastError());
    return HOGATT_OK;
}

template <class T>
int launch_all(const KernelArgs& args, const Resolved& r, int dev, int smem_optin, int grid, cudaStream_t stream,
               const void* q_rot = nullptr) {
    int rc;
    if (r.kernel == HOGATT_KERNEL_DENSE) {
        rc = launch_dense<T>(args, q_rot, std::is_same<T, __half>::value ? HOGATT_F16 : HOGATT_BF16, dev, smem_optin, grid, stream);
    } else if (r.kernel == HOGATT_KERNEL_MMA) {
        bool ef = r.row_blocks == 1;             // every K/V byte is read once: do not let it displace L2 contents
#ifdef HOGATT_EXPERIMENT
        if (getenv("HOGATT_STREAM_ONLY")) return launch_mma_dims<T>(args, args.F, args.E, r.mt, dev, smem_optin,
                                                                    r.cluster > 1 ? r.units * r.cluster : grid, r.cluster, ef, stream, 2);
#endif
        if (r.cluster > 1)      // the cluster kernel merges by itself
            return launch_mma_dims<T>(args, args.F, args.E, r.mt, dev, smem_optin, r.units * r.cluster, r.cluster, ef, stream);
        rc = launch_mma_dims<T>(args, args.F, args.E, r.mt, dev, smem_optin, grid, 0, ef, stream);
    } else {
        rc = launch_fma_dims<T>(args, dev, smem_optin, grid, stream);
    }
    if (rc != HOGATT_OK) return rc;
#ifdef HOGATT_EXPERIMENT
    if (getenv("HOGATT_SKIP_MERGE")) return HOGATT_OK;
#endif
    return launch_merge<T>(args, r, stream);
}

template <>
int launch_all<float>(const KernelArgs& args, const Resolved& r, int dev, int smem_optin, int grid, cudaStream_t stream,
                      const void*) {
    int rc = launch_fma_dims<float>(args, dev, smem_optin, grid, stream);
    if (rc != HOGATT_OK) return rc;
    return launch_merge<float>(args, r, stream);
}

bool aligned16(const void* p) { return ((uintptr_t)p & 15u) == 0; }

int rope_launch(void* rq, const void* queries, const float* cosines, const float* sines, int F, int W, int Hq, int S, int E,
                int rotary_dim, int dtype, cudaStream_t stream) {
    const int64_t rows = (int64_t)F * W * Hq * S;
    if (rows > (1 << 30) || rows * std::max(E, 8) >= ((int64_t)1 << 31)) return HOGATT_ERR_TOO_LARGE;   // 32-bit element counts
    const int64_t work = rows * ((dtype != HOGATT_F32 && E % 8 == 0) ? E / 8 : E);      // chunks or channels
    if (dtype != HOGATT_F32 && rotary_dim == E && E % 16 == 0 && aligned16(cosines) && aligned16(sines) && aligned16(queries) &&
        aligned16(rq)) {
        // whole head rotated: a thread per pair of partner chunks, tables kept in registers over kRopeHeads heads
        const int64_t items = (int64_t)F * W * S * (E / 16);
        const dim3 grid((unsigned)((items + 127) / 128), (unsigned)ceil_div(Hq, kRopeHeads));
        if (dtype == HOGATT_F16)
            rope_pairs_kernel<__half><<<grid, 128, 0, stream>>>((__half*)rq, (const __half*)queries, cosines, sines, F, W, Hq, S, E);
        else
            rope_pairs_kernel<__nv_bfloat16><<<grid, 128, 0, stream>>>((__nv_bfloat16*)rq, (const __nv_bfloat16*)queries, cosines, sines, F, W, Hq, S, E);
        HOGATT_CUDA_OK(cudaGetLastError());
        return HOGATT_OK;
    }
    // one pass of four chunks per thread where there is enough work: 16 CTAs of 128 threads per SM
    int dev = 0, sms = 0, smem_optin = 0;
    if (const int rc = current_device_info(&dev, &sms, &smem_optin)) return rc;
    const unsigned blocks = (unsigned)std::min<int64_t>((work + 127) / 128, (int64_t)sms * 16);
    switch (dtype) {
        case HOGATT_F32:
            rope_kernel<float><<<blocks, 128, 0, stream>>>((float*)rq, (const float*)queries, cosines, sines, F, W, Hq, S, E, rotary_dim);
            break;
        case HOGATT_F16:
            rope_kernel<__half><<<blocks, 128, 0, stream>>>((__half*)rq, (const __half*)queries, cosines, sines, F, W, Hq, S, E, rotary_dim);
            break;
        case HOGATT_BF16:
            rope_kernel<__nv_bfloat16><<<blocks, 128, 0, stream>>>((__nv_bfloat16*)rq, (const __nv_bfloat16*)queries, cosines, sines, F, W, Hq, S, E, rotary_dim);
            break;
        default: return HOGATT_ERR_UNSUPPORTED_DTYPE;
    }
    HOGATT_CUDA_OK(cudaGetLastError());
    return HOGATT_OK;
}

int attention_launch(const hogatt_problem* p, bool fused, cudaStream_t stream, const hogatt_peers* peers = nullptr) {
    Resolved r;
    int rc = resolve(p, &r);
    if (rc != HOGATT_OK) return rc;
    if ((!p->out && !peers) || !p->queries || !p->locations || !p->key_fragments || !p->value_fragments ||
        !p->fragment_rows || !p->workspace)
        return HOGATT_ERR_NULL_POINTER;
    if (peers) {
        if (peers->world < 1 || peers->world > HOGATT_MAX_PEERS || peers->rank < 0 || peers->rank >= peers->world)
            return HOGATT_ERR_BAD_SHAPE;
        for (int i = 0; i < peers->world; ++i) {
            if (!peers->out_full[i] || !peers->flags[i]) return HOGATT_ERR_NULL_POINTER;
            if (!aligned16(peers->out_full[i]) || ((uintptr_t)peers->flags[i] & 3u)) return HOGATT_ERR_MISALIGNED;
        }
    }
    if (fused) {
        if (!p->cosines || !p->sines) return HOGATT_ERR_NULL_POINTER;
        if (p->rotary_dim <= 0 || p->rotary_dim > p->E || (p->rotary_dim & 1)) return HOGATT_ERR_BAD_SHAPE;
    } else if (p->cosines || p->sines || p->rq) {
        return HOGATT_ERR_BAD_SHAPE;      // pre-rotated queries: nothing to rotate, nothing to write back
    }
    const size_t sz = dtype_size(p->dtype);
    if ((p->E * sz) % 16 != 0 || (p->Ev * sz) % 16 != 0) return HOGATT_ERR_UNSUPPORTED_HEAD_DIM;
    if ((!peers && !aligned16(p->out)) || !aligned16(p->queries) || !aligned16(p->workspace) || ((uintptr_t)p->workspace & 255u))
        return HOGATT_ERR_MISALIGNED;
    if (p->rq && !aligned16(p->rq)) return HOGATT_ERR_MISALIGNED;
    if (fused && (((uintptr_t)p->cosines & 3u) || ((uintptr_t)p->sines & 3u))) return HOGATT_ERR_MISALIGNED;

    int dev, sms, smem_optin;
    rc = current_device_info(&dev, &sms, &smem_optin);
    if (rc != HOGATT_OK) return rc;
    const int grid = grid_size(p, sms);
    refine_row_blocks(p, &r, grid, tiles_upper_bound(p, r));
    const WorkspaceLayout w = carve(p, r, grid);
    if (p->workspace_bytes < w.total) return HOGATT_ERR_WORKSPACE_TOO_SMALL;
    r.cluster = choose_cluster(p, r, dev, sms, smem_optin, tiles_upper_bound(p, r));
    if (r.cluster_forced && r.cluster == 0) return HOGATT_ERR_BAD_KERNEL_CHOICE;

    KernelArgs args;
    memset(&args, 0, sizeof(args));
    args.F = p->F; args.W = p->W; args.Hq = p->Hq; args.Hkv = p->Hkv; args.G = p->Hq / p->Hkv;
    args.E = p->E; args.Ev = p->Ev; args.S = p->S; args.R = fused ? p->rotary_dim : 0;
    args.rows_total = p->W * args.G * p->S;
    args.rows_per_block = r.rows_per_block;
    args.row_blocks = r.row_blocks;
    args.parts_per_unit = w.parts;
    args.l2scale = p->scale * 1.4426950408889634f;
    args.out = p->out;
    args.rq = fused ? p->rq : nullptr;
    args.q = p->queries;
    args.cos = fused ? p->cosines : nullptr;
    args.sin = fused ? p->sines : nullptr;
    args.loc = p->locations;
    args.flen = p->fragment_lengths;
    unsigned char* ws = static_cast<unsigned char*>(p->workspace);
    args.header = reinterpret_cast<int*>(ws + w.header);
    args.ws_o = reinterpret_cast<float*>(ws + w.o);
    args.ws_m = reinterpret_cast<float*>(ws + w.m);
    args.ws_l = reinterpret_cast<float*>(ws + w.l);
    args.status = p->device_status;
#ifdef HOGATT_TIMELINE
    {
        static std::atomic<int> trace_counter{0};
    args.debug_id = trace_counter.fetch_add(1) % kTraceCalls;
    }
#endif
    if (peers) {
        args.world = peers->world;
        args.rank = peers->rank;
        for (int i = 0; i < peers->world; ++i) args.peer_out[i] = peers->out_full[i];
    }
    // Host plan: only the tensor-core kernel takes one (the FMA kernel always derives its tiles on the device).
    const bool host_plan = p->host_lengths != nullptr && (r.kernel == HOGATT_KERNEL_MMA || r.kernel == HOGATT_KERNEL_DENSE) &&
                           !host_plan_disabled();
    int64_t plan_tiles = 0;
    for (int f = 0; f < p->F; ++f) {
        const int rows = p->fragment_rows[f];
        if (rows < 0) return HOGATT_ERR_BAD_SHAPE;
        if (rows > 0 && (!p->key_fragments[f] || !p->value_fragments[f])) return HOGATT_ERR_NULL_POINTER;
        if (!aligned16(p->key_fragments[f]) || !aligned16(p->value_fragments[f])) return HOGATT_ERR_MISALIGNED;
        args.ft.e[f].k = p->key_fragments[f];
        args.ft.e[f].v = p->value_fragments[f];
        args.ft.e[f].rows = rows;
        args.ft.e[f].vis = host_plan ? std::max(0, std::min(rows, p->host_lengths[f])) : 0;
        plan_tiles += ceil_div(args.ft.e[f].vis, r.tile_tokens);
    }
    if (host_plan) {
        if (plan_tiles * r.units > ((int64_t)1 << 40) || plan_tiles > (1 << 30)) return HOGATT_ERR_TOO_LARGE;
        args.host_plan = 1;
        args.plan_tiles = (int)plan_tiles;
        args.plan_ctas = effective_ctas(plan_tiles * r.units, grid);
        if (r.kernel == HOGATT_KERNEL_MMA) {         // ranges that stay inside one fragment of one unit, where the lengths allow
            int pre[HOGATT_MAX_FRAGMENTS + 1];
            pre[0] = 0;
            for (int f = 0; f < p->F; ++f) pre[f + 1] = pre[f] + ceil_div(args.ft.e[f].vis, r.tile_tokens);
            args.plan_ctas = aligned_ctas(pre, p->F, r.units, grid);
        }
        args.stable_fragments = pdl_enabled() ? std::max(0, std::min(p->F, p->stable_fragments)) : 0;
    }

    // The tcgen05 kernel takes its queries already rotated, from memory: the rotated-query output of the call (or
    // room in the workspace when the caller does not want it) is written by the stand-alone rotation kernel first.
    const void* q_rot = p->queries;
    if (r.kernel == HOGATT_KERNEL_DENSE && fused) {
        void* dst = p->rq ? p->rq : static_cast<void*>(ws + w.rq);
        rc = rope_launch(dst, p->queries, p->cosines, p->sines, p->F, p->W, p->Hq, p->S, p->E, p->rotary_dim, p->dtype, stream);
        if (rc != HOGATT_OK) return rc;
        q_rot = dst;
    }
    switch (p->dtype) {
        case HOGATT_F32: rc = launch_all<float>(args, r, dev, smem_optin, grid, stream, nullptr); break;
        case HOGATT_F16: rc = launch_all<__half>(args, r, dev, smem_optin, grid, stream, q_rot); break;
        case HOGATT_BF16: rc = launch_all<__nv_bfloat16>(args, r, dev, smem_optin, grid, stream, q_rot); break;
        default: return HOGATT_ERR_UNSUPPORTED_DTYPE;
    }
    if (rc != HOGATT_OK || !peers) return rc;
    PeerFlags pf;
    memset(&pf, 0, sizeof(pf));
    for (int i = 0; i < peers->world; ++i) pf.f[i] = peers->flags[i];
    HOGATT_CUDA_OK(launch_kernel(gather_signal_kernel, dim3(1), dim3(32), 0, stream, pf, (int)peers->world, (int)peers->rank,
                                 p->device_status, (int)args.debug_id));
    return HOGATT_OK;
}

// ---- paged variants ----------------------------------------------------------------------------------

struct PagedPlan {
    int tokens_per_group, head_blocks, groups_bound, units, splits;
    size_t o, m, l, total;
};

int plan_paged(const hogatt_paged_problem* p, int sms, PagedPlan* pl) {
    if (p == nullptr) return HOGATT_ERR_NULL_POINTER;
    const bool packed = p->cu_seqlens_q != nullptr;
    if (p->F <= 0 || p->W <= 0 || p->Hq <= 0 || p->Hkv <= 0 || p->E <= 0 || p->Ev <= 0 || p->block_size <= 0 ||
        p->max_blocks_per_seq <= 0 || p->Hq % p->Hkv != 0 || (packed ? p->total_q_tokens < 0 : p->S <= 0))
        return HOGATT_ERR_BAD_SHAPE;
    if (p->dtype != HOGATT_F32 && p->dtype != HOGATT_F16 && p->dtype != HOGATT_BF16) return HOGATT_ERR_UNSUPPORTED_DTYPE;
    if (p->F > 4096) return HOGATT_ERR_TOO_MANY_FRAGMENTS;
    const int vec = 16 / (int)dtype_size(p->dtype);
    if ((p->Ev != 32 && p->Ev != 64 && p->Ev != 128 && p->Ev != 256) || p->E > 256 || p->E % vec != 0)
        return HOGATT_ERR_UNSUPPORTED_HEAD_DIM;
    const int G = p->Hq / p->Hkv;
    pl->tokens_per_group = G >= 16 ? 1 : 16 / G;
    pl->head_blocks = (G + 15) / 16;
    const int64_t groups = packed ? ((int64_t)p->total_q_tokens + pl->tokens_per_group - 1) / pl->tokens_per_group + p->W
                                  : (int64_t)p->W * ((p->S + pl->tokens_per_group - 1) / pl->tokens_per_group);
    const int64_t units = groups * pl->head_blocks * p->Hkv;
    if (units > (1 << 24)) return HOGATT_ERR_TOO_LARGE;
    pl->groups_bound = (int)groups;
    pl->units = (int)std::max<int64_t>(units, 1);
    // at most 24 partials per row: what the merge step fetches in one round trip
    // and CTAs for three per SM (what registers and shared memory of the tensor-core kernel allow; measured 36.7 us
    // with two per SM, 34.7 with three, at 8 sequences x 16 K keys)
    pl->splits = std::max(1, std::min(24, (3 * sms + pl->units - 1) / pl->units));
    const size_t slots = (size_t)pl->units * pl->splits * kFmaRows;
    pl->o = 0;
    pl->m = pl->o + align_up(slots * p->Ev * sizeof(float), 256);
    pl->l = pl->m + align_up(slots * sizeof(float), 256);
    pl->total = pl->l + align_up(slots * sizeof(float), 256);
    return HOGATT_OK;
}

template <class T, int EV>
int launch_paged(const PagedArgs& a, const PagedPlan& pl, int dev, int smem_optin, cudaStream_t stream) {
    static std::atomic<size_t> granted[kMaxDevices];
    const size_t smem = paged_smem_bytes(a.E, EV, a.F);
    if (smem > (size_t)smem_optin) return HOGATT_ERR_TOO_MANY_FRAGMENTS;
    int rc = ensure_smem_limit(paged_attention_kernel<T, EV>, dev, smem, granted);
    if (rc != HOGATT_OK) return rc;
    paged_attention_kernel<T, EV><<<dim3(pl.units, pl.splits), kFmaThreads, smem, stream>>>(a);
    HOGATT_CUDA_OK(cudaGetLastError());
    paged_merge_kernel<T><<<dim3(pl.units, kFmaRows / kMergeWarps), kMergeWarps * 32, 0, stream>>>(a);
    HOGATT_CUDA_OK(cudaGetLastError());
    return HOGATT_OK;
}

// HOGATT_PAGED_MMA=0 in the environment keeps AUTO on the CUDA-core paged kernel (A/B measurements).
bool paged_mma_disabled() {
    static const bool off = [] {
        const char* v = getenv("HOGATT_PAGED_MMA");
        return v && v[0] == '0';
    }();
    return off;
}

// Two ring stages: measured best at 8 sequences x 16 K keys (deeper rings cost resident CTAs: three stages 53 us
// against 40).
template <class T, int HD>
int launch_paged_mma(const PagedArgs& a, const PagedPlan& pl, int dev, int smem_optin, cudaStream_t stream) {
    static std::atomic<size_t> granted[kMaxDevices];
    const size_t smem = paged_mma_smem_bytes<HD>(a.F);
    if (smem > (size_t)smem_optin) return HOGATT_ERR_TOO_MANY_FRAGMENTS;
    int rc = ensure_smem_limit(paged_mma_kernel<T, HD>, dev, smem, granted);
    if (rc != HOGATT_OK) return rc;
    HOGATT_CUDA_OK(launch_kernel(paged_mma_kernel<T, HD>, dim3(pl.units, pl.splits), dim3(PagedMmaCfg<HD>::THREADS), smem, stream, a));
    HOGATT_CUDA_OK(launch_kernel(paged_merge_kernel<T>, dim3(pl.units, kFmaRows / kMergeWarps), dim3(kMergeWarps * 32), 0, stream, a));
    return HOGATT_OK;
}

template <class T>
bool paged_mma_eligible(const PagedArgs& a) {
    return !std::is_same<T, float>::value && a.E == a.Ev && (a.E == 64 || a.E == 128);
}

template <class T>
int launch_paged_dims(const PagedArgs& a, const PagedPlan& pl, int kernel, int dev, int smem_optin, cudaStream_t stream) {
    if (kernel != HOGATT_KERNEL_AUTO && kernel != HOGATT_KERNEL_FMA && kernel != HOGATT_KERNEL_MMA) return HOGATT_ERR_BAD_KERNEL_CHOICE;
    if (kernel == HOGATT_KERNEL_MMA && !paged_mma_eligible<T>(a)) return HOGATT_ERR_BAD_KERNEL_CHOICE;
    if constexpr (!std::is_same<T, float>::value) {
        if (kernel == HOGATT_KERNEL_MMA || (kernel == HOGATT_KERNEL_AUTO && paged_mma_eligible<T>(a) && !paged_mma_disabled()))
            return a.E == 128 ? launch_paged_mma<T, 128>(a, pl, dev, smem_optin, stream)
                              : launch_paged_mma<T, 64>(a, pl, dev, smem_optin, stream);
    }
    switch (a.Ev) {
        case 32: return launch_paged<T, 32>(a, pl, dev, smem_optin, stream);
        case 64: return launch_paged<T, 64>(a, pl, dev, smem_optin, stream);
        case 128: return launch_paged<T, 128>(a, pl, dev, smem_optin, stream);
        case 256: return launch_paged<T, 256>(a, pl, dev, smem_optin, stream);
    }
    return HOGATT_ERR_UNSUPPORTED_HEAD_DIM;
}

// ---- fixed scratch for hogatt_fused_launch_static ---------------------------------------------------
// In host code `g_static_scratch` is only a handle for the symbol, not a device address; the address
// the kernels can use comes from cudaGetSymbolAddress, looked up once per device.
static __device__ __align__(256) unsigned char g_static_scratch[HOGATT_STATIC_SCRATCH_BYTES];
std::atomic<void*> g_static_scratch_ptr[kMaxDevices];

int static_scratch_for_current_device(void** out) {
    int dev = -1;
    HOGATT_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return HOGATT_ERR_CUDA;
    void* ptr = g_static_scratch_ptr[dev].load(std::memory_order_acquire);
    if (ptr == nullptr) {
        HOGATT_CUDA_OK(cudaGetSymbolAddress(&ptr, g_static_scratch));     // device `dev` is current
        if (ptr == nullptr) return HOGATT_ERR_CUDA;
        g_static_scratch_ptr[dev].store(ptr, std::memory_order_release);
    }
    *out = ptr;
    return HOGATT_OK;
}

}  // namespace
}  // namespace hogatt

using namespace hogatt;

extern "C" {

int hogatt_abi_version(void) { return HOGATT_ABI_VERSION; }

const char* hogatt_status_string(int status) {
    switch (status) {
        case HOGATT_OK: return "ok";
        case HOGATT_ERR_NULL_POINTER: return "a required pointer is NULL";
        case HOGATT_ERR_BAD_SHAPE: return "bad shape (non-positive dim, Hq not a multiple of Hkv, bad rotary_dim, or rope arguments on the pre-rotated entry point)";
        case HOGATT_ERR_UNSUPPORTED_HEAD_DIM: return "unsupported head size (rows must be multiples of 16 bytes; E <= 256; Ev in {32,64,128,256})";
        case HOGATT_ERR_UNSUPPORTED_DTYPE: return "unsupported dtype (f32, f16, bf16)";
        case HOGATT_ERR_TOO_MANY_FRAGMENTS: return "too many fragments (HOGATT_MAX_FRAGMENTS)";
        case HOGATT_ERR_MISALIGNED: return "a tensor does not start on a 16-byte boundary (workspace: 256)";
        case HOGATT_ERR_WORKSPACE_TOO_SMALL: return "workspace smaller than hogatt_workspace_bytes()";
        case HOGATT_ERR_CUDA: return "a CUDA runtime call failed (hogatt_last_cuda_error())";
        case HOGATT_ERR_BAD_KERNEL_CHOICE: return "the requested kernel cannot run this dtype / head size";
        case HOGATT_ERR_TOO_LARGE: return "problem too large for 32-bit row indexing";
        case HOGATT_ERR_EXCEEDS_STATIC_SCRATCH: return "problem needs more scratch than the fixed HOGATT_STATIC_SCRATCH_BYTES array of hogatt_fused_launch_static; use hogatt_fused_launch with a caller workspace";
    }
    return "unknown status";
}

int hogatt_last_cuda_error(void) { return tl_last_cuda_error; }

size_t hogatt_workspace_bytes(const hogatt_problem* p) {
    Resolved r;
    if (resolve(p, &r) != HOGATT_OK) return 0;
    int dev, sms, smem_optin;
    if (current_device_info(&dev, &sms, &smem_optin) != HOGATT_OK) return 0;
    const int grid = grid_size(p, sms);
    size_t need = carve(p, r, grid).total;
    if (r.kernel == HOGATT_KERNEL_MMA && !r.cluster_forced) {
        // a launch may cut the query rows into smaller blocks than resolve() did (refine_row_blocks): room for any of them
        const int64_t rows_total = (int64_t)p->W * (p->Hq / p->Hkv) * p->S;
        for (int mt = 1; mt < r.mt; mt *= 2) {
            Resolved q = r;
            q.mt = mt;
            q.rows_per_block = 16 * mt;
            q.row_blocks = (int)((rows_total + q.rows_per_block - 1) / q.rows_per_block);
            q.units = q.row_blocks * p->Hkv;
            need = std::max(need, carve(p, q, grid).total);
        }
    }
    return need;
}

int hogatt_sdpa_launch(const hogatt_problem* p, hogatt_stream_t stream) {
    return attention_launch(p, /*fused=*/false, reinterpret_cast<cudaStream_t>(stream));
}

int hogatt_fused_launch(const hogatt_problem* p, hogatt_stream_t stream) {
    return attention_launch(p, /*fused=*/true, reinterpret_cast<cudaStream_t>(stream));
}

int hogatt_fused_launch_static(const hogatt_problem* p, hogatt_stream_t stream) {
    if (p == nullptr) return HOGATT_ERR_NULL_POINTER;
    const size_t need = hogatt_workspace_bytes(p);
    if (need == 0) {                         // let the regular path name what is wrong with the problem
        Resolved r;
        const int rc = resolve(p, &r);
        return rc != HOGATT_OK ? rc : HOGATT_ERR_CUDA;
    }
    if (need > (size_t)HOGATT_STATIC_SCRATCH_BYTES) return HOGATT_ERR_EXCEEDS_STATIC_SCRATCH;
    void* scratch = nullptr;
    const int rc = static_scratch_for_current_device(&scratch);
    if (rc != HOGATT_OK) return rc;
    hogatt_problem q = *p;
    q.workspace = scratch;
    q.workspace_bytes = HOGATT_STATIC_SCRATCH_BYTES;
    return attention_launch(&q, /*fused=*/true, reinterpret_cast<cudaStream_t>(stream));
}

size_t hogatt_paged_workspace_bytes(const hogatt_paged_problem* p) {
    int dev, sms, smem_optin;
    if (current_device_info(&dev, &sms, &smem_optin) != HOGATT_OK) return 0;
    PagedPlan pl;
    if (plan_paged(p, sms, &pl) != HOGATT_OK) return 0;
    return pl.total;
}

int hogatt_paged_sdpa_launch(const hogatt_paged_problem* p, hogatt_stream_t stream_) {
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    int dev, sms, smem_optin;
    int rc = current_device_info(&dev, &sms, &smem_optin);
    if (rc != HOGATT_OK) return rc;
    PagedPlan pl;
    rc = plan_paged(p, sms, &pl);
    if (rc != HOGATT_OK) return rc;
    if (!p->out || !p->queries || !p->locations || !p->fragment_lengths || !p->key_cache || !p->value_cache ||
        !p->block_table || !p->workspace)
        return HOGATT_ERR_NULL_POINTER;
    if (!aligned16(p->out) || !aligned16(p->queries) || !aligned16(p->key_cache) || !aligned16(p->value_cache) ||
        ((uintptr_t)p->workspace & 255u))
        return HOGATT_ERR_MISALIGNED;
    if (p->workspace_bytes < pl.total) return HOGATT_ERR_WORKSPACE_TOO_SMALL;
    const bool packed = p->cu_seqlens_q != nullptr;
    if (packed && p->total_q_tokens == 0) return HOGATT_OK;

    PagedArgs a;
    memset(&a, 0, sizeof(a));
    a.F = p->F; a.W = p->W; a.Hq = p->Hq; a.Hkv = p->Hkv; a.G = p->Hq / p->Hkv; a.E = p->E; a.Ev = p->Ev;
    a.S = p->S; a.total_q = packed ? p->total_q_tokens : p->W * p->S;
    a.block_size = p->block_size; a.max_blocks = p->max_blocks_per_seq;
    a.tokens_per_group = pl.tokens_per_group; a.head_blocks = pl.head_blocks; a.groups_bound = pl.groups_bound;
    a.splits = pl.splits;
    a.l2scale = p->scale * 1.4426950408889634f;
    if (packed) {     // q [F,total_q,Hq,E], out [total_q,Hq,Ev], loc [F,total_q], len [F,W]; s is the packed token index
        a.q_f = (long long)a.total_q * p->Hq * p->E; a.q_w = 0; a.q_s = (long long)p->Hq * p->E; a.q_h = p->E;
        a.o_w = 0; a.o_s = (long long)p->Hq * p->Ev; a.o_h = p->Ev;
        a.loc_f = a.total_q; a.loc_w = 0; a.len_f = p->W; a.len_w = 1;
    } else {          // q [F,W,Hq,S,E], out [W,Hq,S,Ev], loc [F,W,S], len [F]
        a.q_f = (long long)p->W * p->Hq * p->S * p->E; a.q_w = (long long)p->Hq * p->S * p->E; a.q_s = p->E;
        a.q_h = (long long)p->S * p->E;
        a.o_w = (long long)p->Hq * p->S * p->Ev; a.o_s = p->Ev; a.o_h = (long long)p->S * p->Ev;
        a.loc_f = p->W * p->S; a.loc_w = p->S; a.len_f = 1; a.len_w = 0;
    }
    a.out = p->out; a.q = p->queries; a.loc = p->locations; a.flen = p->fragment_lengths;
    a.kcache = p->key_cache; a.vcache = p->value_cache; a.block_table = p->block_table; a.cu_seqlens = p->cu_seqlens_q;
    unsigned char* ws = static_cast<unsigned char*>(p->workspace);
    a.ws_o = reinterpret_cast<float*>(ws + pl.o);
    a.ws_m = reinterpret_cast<float*>(ws + pl.m);
    a.ws_l = reinterpret_cast<float*>(ws + pl.l);
    switch (p->dtype) {
        case HOGATT_F32: return launch_paged_dims<float>(a, pl, p->kernel, dev, smem_optin, stream);
        case HOGATT_F16: return launch_paged_dims<__half>(a, pl, p->kernel, dev, smem_optin, stream);
        case HOGATT_BF16: return launch_paged_dims<__nv_bfloat16>(a, pl, p->kernel, dev, smem_optin, stream);
    }
    return HOGATT_ERR_UNSUPPORTED_DTYPE;
}

int hogatt_copy_to_blocks_launch(const void* key_states, const void* value_states, void* key_cache, void* value_cache,
                                 const int32_t* block_table, const int32_t* seq_lengths, int32_t B, int32_t Hkv,
                                 int32_t S_new, int32_t E, int32_t Ev, int32_t block_size, int32_t max_blocks,
                                 int32_t dtype, hogatt_stream_t stream_) {
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    if (!key_states || !value_states || !key_cache || !value_cache || !block_table || !seq_lengths) return HOGATT_ERR_NULL_POINTER;
    if (B <= 0 || Hkv <= 0 || S_new < 0 || E <= 0 || Ev <= 0 || block_size <= 0 || max_blocks <= 0) return HOGATT_ERR_BAD_SHAPE;
    if (dtype != HOGATT_F32 && dtype != HOGATT_F16 && dtype != HOGATT_BF16) return HOGATT_ERR_UNSUPPORTED_DTYPE;
    const int vec = 16 / (int)dtype_size(dtype);
    if (E % vec != 0 || Ev % vec != 0) return HOGATT_ERR_UNSUPPORTED_HEAD_DIM;
    if (!aligned16(key_states) || !aligned16(value_states) || !aligned16(key_cache) || !aligned16(value_cache)) return HOGATT_ERR_MISALIGNED;
    if (S_new == 0) return HOGATT_OK;
    const int64_t total = (int64_t)B * Hkv * S_new * ((E + Ev) / vec);
    int dev = 0, sms = 0, smem_optin = 0;
    if (const int rc = current_device_info(&dev, &sms, &smem_optin)) return rc;
    const unsigned blocks = (unsigned)std::min<int64_t>((total + 255) / 256, (int64_t)sms * 8);   // 8 CTAs of 256 threads per SM
    switch (dtype) {
        case HOGATT_F32:
            copy_to_blocks_kernel<float><<<blocks, 256, 0, stream>>>((const float*)key_states, (const float*)value_states, (float*)key_cache, (float*)value_cache, block_table, seq_lengths, B, Hkv, S_new, E, Ev, block_size, max_blocks);
            break;
        case HOGATT_F16:
            copy_to_blocks_kernel<__half><<<blocks, 256, 0, stream>>>((const __half*)key_states, (const __half*)value_states, (__half*)key_cache, (__half*)value_cache, block_table, seq_lengths, B, Hkv, S_new, E, Ev, block_size, max_blocks);
            break;
        default:
            copy_to_blocks_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)key_states, (const __nv_bfloat16*)value_states, (__nv_bfloat16*)key_cache, (__nv_bfloat16*)value_cache, block_table, seq_lengths, B, Hkv, S_new, E, Ev, block_size, max_blocks);
            break;
    }
    HOGATT_CUDA_OK(cudaGetLastError());
    return HOGATT_OK;
}

int hogatt_fused_launch_gather(const hogatt_problem* p, const hogatt_peers* peers, hogatt_stream_t stream) {
    if (peers == nullptr) return HOGATT_ERR_NULL_POINTER;
    return attention_launch(p, /*fused=*/true, reinterpret_cast<cudaStream_t>(stream), peers);
}

int hogatt_rope_launch(void* rq, const void* queries, const float* cosines, const float* sines, int32_t F, int32_t W,
                       int32_t Hq, int32_t S, int32_t E, int32_t rotary_dim, int32_t dtype, hogatt_stream_t stream_) {
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    if (!rq || !queries || !cosines || !sines) return HOGATT_ERR_NULL_POINTER;
    if (F <= 0 || W <= 0 || Hq <= 0 || S <= 0 || E <= 0 || rotary_dim <= 0 || rotary_dim > E || (rotary_dim & 1))
        return HOGATT_ERR_BAD_SHAPE;
    if (dtype != HOGATT_F32 && dtype != HOGATT_F16 && dtype != HOGATT_BF16) return HOGATT_ERR_UNSUPPORTED_DTYPE;
    return rope_launch(rq, queries, cosines, sines, F, W, Hq, S, E, rotary_dim, dtype, stream);
}

#ifdef HOGATT_TIMELINE
// Debug builds only: copy out the timeline of the instrumented CTA (see hogatt_device.cuh).
int hogatt_debug_read_timeline(long long* times /*[2][1024]*/, int* tags /*[2][1024]*/, int* counts /*[2]*/) {
    HOGATT_CUDA_OK(cudaMemcpyFromSymbol(times, g_timeline, sizeof(long long) * 2048));
    HOGATT_CUDA_OK(cudaMemcpyFromSymbol(tags, g_timeline_tag, sizeof(int) * 2048));
    HOGATT_CUDA_OK(cudaMemcpyFromSymbol(counts, g_timeline_n, sizeof(int) * 2));
    return HOGATT_OK;
}
int hogatt_debug_cta_times(unsigned long long* out /*[3][256]*/, unsigned int* sm /*[256]*/) {
    HOGATT_CUDA_OK(cudaMemcpyFromSymbol(out, g_cta_t, sizeof(unsigned long long) * 768));
    HOGATT_CUDA_OK(cudaMemcpyFromSymbol(sm, g_cta_sm, sizeof(unsigned int) * 256));
    return HOGATT_OK;
}
// out [kTraceCalls][kTraceEvents][256], mout [kTraceCalls][2]; reset != 0 re-arms the merge kernel's min / max slots
int hogatt_debug_trace(unsigned long long* out, unsigned long long* mout, int reset) {
    HOGATT_CUDA_OK(cudaMemcpyFromSymbol(out, g_trace, sizeof(g_trace)));
    HOGATT_CUDA_OK(cudaMemcpyFromSymbol(mout, g_mtrace, sizeof(g_mtrace)));
    if (reset) {
        static unsigned long long init[kTraceCalls][2];
        for (int i = 0; i < kTraceCalls; ++i) {
            init[i][0] = ~0ull;
            init[i][1] = 0;
        }
        HOGATT_CUDA_OK(cudaMemcpyToSymbol(g_mtrace, init, sizeof(init)));
    }
    return HOGATT_OK;
}
int hogatt_debug_mphase(unsigned long long* out) {
    HOGATT_CUDA_OK(cudaMemcpyFromSymbol(out, g_mphase, sizeof(g_mphase)));
    return HOGATT_OK;
}
int hogatt_debug_strace(unsigned long long* out) {
    HOGATT_CUDA_OK(cudaMemcpyFromSymbol(out, g_strace, sizeof(g_strace)));
    return HOGATT_OK;
}
int hogatt_debug_spans(unsigned long long* out8, int reset) {
    HOGATT_CUDA_OK(cudaMemcpyFromSymbol(out8, g_span, sizeof(unsigned long long) * 8));
    if (reset) {
        unsigned long long init[8] = {~0ull, 0, ~0ull, 0, ~0ull, 0, ~0ull, 0};
        HOGATT_CUDA_OK(cudaMemcpyToSymbol(g_span, init, sizeof(init)));
    }
    return HOGATT_OK;
}
#endif

int hogatt_plan_describe(const hogatt_problem* p, const int32_t* visible_rows, int32_t num_sms, int32_t plan[8]) {
    Resolved r;
    int rc = resolve(p, &r);
    if (rc != HOGATT_OK) return rc;
    if (!visible_rows || !plan) return HOGATT_ERR_NULL_POINTER;
    if (num_sms <= 0) return HOGATT_ERR_BAD_SHAPE;
    int64_t th = 0;
    for (int f = 0; f < p->F; ++f) th += ceil_div(visible_rows[f] < 0 ? 0 : visible_rows[f], r.tile_tokens);
    if (th > (1 << 30)) return HOGATT_ERR_TOO_LARGE;
    const int grid = grid_size(p, num_sms);
    refine_row_blocks(p, &r, grid, th);
    const int cluster = r.cluster_forced ? cluster_upper_bound(r, num_sms) : 0;
    if (r.cluster_forced && cluster == 0) return HOGATT_ERR_BAD_KERNEL_CHOICE;
    plan[0] = r.tile_tokens;
    plan[1] = r.rows_per_block;
    plan[2] = r.row_blocks;
    plan[3] = (int)th;
    plan[4] = r.units;
    plan[5] = cluster ? r.units * cluster : effective_ctas((int64_t)r.units * th, grid);
    if (!cluster && r.kernel == HOGATT_KERNEL_MMA) {
        int pre[HOGATT_MAX_FRAGMENTS + 1];
        pre[0] = 0;
        for (int f = 0; f < p->F; ++f) pre[f + 1] = pre[f] + ceil_div(visible_rows[f] < 0 ? 0 : visible_rows[f], r.tile_tokens);
        plan[5] = aligned_ctas(pre, p->F, r.units, grid);
    }
    plan[6] = cluster ? cluster : max_parts_per_unit(r.units, grid);
    plan[7] = cluster ? HOGATT_KERNEL_MMA_CLUSTER : r.kernel;
    return HOGATT_OK;
}

int hogatt_step_plan_launch(const hogatt_step_plan* p, hogatt_stream_t stream) {
    if (!p) return HOGATT_ERR_NULL_POINTER;
    if (!p->order || !p->fragment_lengths || !p->inv_freq || !p->locations || !p->cosines || !p->sines)
        return HOGATT_ERR_NULL_POINTER;
    if (p->F <= 0 || p->W <= 0 || p->S <= 0 || p->rotary_dim <= 0 || (p->rotary_dim & 1)) return HOGATT_ERR_BAD_SHAPE;
    if (p->F > HOGATT_MAX_FRAGMENTS) return HOGATT_ERR_TOO_MANY_FRAGMENTS;
    if ((int64_t)p->F * p->W > (1 << 24) || (int64_t)p->F * p->W * p->S > (1 << 26)) return HOGATT_ERR_TOO_LARGE;
    if (p->round_tables_to != HOGATT_F32 && p->round_tables_to != HOGATT_F16 && p->round_tables_to != HOGATT_BF16)
        return HOGATT_ERR_UNSUPPORTED_DTYPE;
    StepPlanArgs a;
    a.F = p->F; a.W = p->W; a.S = p->S; a.R = p->rotary_dim;
    a.order = p->order; a.lengths = p->fragment_lengths; a.inv_freq = p->inv_freq;
    a.attention_scaling = p->attention_scaling;
    a.round_to = p->round_tables_to;
    a.loc = p->locations; a.cos = p->cosines; a.sin = p->sines;
    step_plan_kernel<<<(unsigned)(p->F * p->W), 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(a);
    HOGATT_CUDA_OK(cudaGetLastError());
    return HOGATT_OK;
}

int hogatt_append_launch(const hogatt_append* p, hogatt_stream_t stream) {
    if (!p) return HOGATT_ERR_NULL_POINTER;
    if (!p->keys || !p->values || !p->cosines || !p->sines || !p->write_to || !p->key_fragments || !p->value_fragments ||
        !p->fragment_rows || !p->lengths_in || !p->lengths_out)
        return HOGATT_ERR_NULL_POINTER;
    if (p->lengths_in == p->lengths_out) return HOGATT_ERR_BAD_SHAPE;
    if (p->W <= 0 || p->W > HOGATT_MAX_APPEND_SOURCES || p->Hkv <= 0 || p->E <= 0 || p->Ev <= 0 || p->S <= 0 || p->F <= 0 ||
        p->rotary_dim <= 0 || p->rotary_dim > p->E || (p->rotary_dim & 1))
        return HOGATT_ERR_BAD_SHAPE;
    if (p->F > HOGATT_MAX_FRAGMENTS) return HOGATT_ERR_TOO_MANY_FRAGMENTS;
    if (p->dtype != HOGATT_F32 && p->dtype != HOGATT_F16 && p->dtype != HOGATT_BF16) return HOGATT_ERR_UNSUPPORTED_DTYPE;
    if (p->table_dtype != HOGATT_F32 && p->table_dtype != p->dtype) return HOGATT_ERR_UNSUPPORTED_DTYPE;
    AppendArgs a;
    memset(&a, 0, sizeof(a));
    a.W = p->W; a.Hkv = p->Hkv; a.E = p->E; a.Ev = p->Ev; a.S = p->S; a.R = p->rotary_dim; a.F = p->F;
    a.tables_lowp = (p->table_dtype != HOGATT_F32) ? 1 : 0;
    a.take_leading = p->take_leading ? 1 : 0;
    a.k = p->keys; a.v = p->values; a.cos = p->cosines; a.sin = p->sines;
    for (int i = 0; i < 3; ++i) {
        a.ks[i] = p->key_strides[i];
        a.vs[i] = p->value_strides[i];
    }
    a.ts[0] = p->table_strides[0]; a.ts[1] = p->table_strides[1];
    a.new_rows = p->new_rows; a.len_in = p->lengths_in; a.len_out = p->lengths_out; a.status = p->device_status;
    for (int w = 0; w < p->W; ++w) {
        if (p->write_to[w] < 0 || p->write_to[w] >= p->F) return HOGATT_ERR_BAD_SHAPE;
        a.write_to[w] = p->write_to[w];
    }
    const size_t sz = dtype_size(p->dtype);
    const int vec = 16 / (int)sz;
    bool vectorised = sz == 2 && p->E % vec == 0 && p->Ev % vec == 0 && aligned16(p->keys) && aligned16(p->values);
    for (int i = 0; i < 3; ++i) vectorised = vectorised && p->key_strides[i] % vec == 0 && p->value_strides[i] % vec == 0;
    if (!a.tables_lowp)           // rotate_chunk reads the fp32 tables eight entries at a time, both halves of the rotation
        vectorised = vectorised && p->rotary_dim % 16 == 0 && aligned16(p->cosines) && aligned16(p->sines) &&
                     p->table_strides[0] % 4 == 0 && p->table_strides[1] % 4 == 0;
    for (int f = 0; f < p->F; ++f) {
        if (p->fragment_rows[f] < 0) return HOGATT_ERR_BAD_SHAPE;
        if (p->fragment_rows[f] > 0 && (!p->key_fragments[f] || !p->value_fragments[f])) return HOGATT_ERR_NULL_POINTER;
        if (!aligned16(p->key_fragments[f]) || !aligned16(p->value_fragments[f])) return HOGATT_ERR_MISALIGNED;
        a.ft.e[f].k = p->key_fragments[f];
        a.ft.e[f].v = p->value_fragments[f];
        a.ft.e[f].rows = p->fragment_rows[f];
    }
    const int64_t pieces = (int64_t)p->S * ((p->E + p->Ev) / (vectorised ? vec : 1));
    dim3 grid((unsigned)std::min<int64_t>((pieces + 255) / 256, 1 << 14), (unsigned)p->Hkv, (unsigned)p->W);
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    switch (p->dtype) {
        case HOGATT_F32: append_kernel<float><<<grid, 256, 0, st>>>(a, 0); break;
        case HOGATT_F16: append_kernel<__half><<<grid, 256, 0, st>>>(a, vectorised ? 1 : 0); break;
        default: append_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(a, vectorised ? 1 : 0); break;
    }
    HOGATT_CUDA_OK(cudaGetLastError());
    return HOGATT_OK;
}

int hogatt_launch_shape(const hogatt_problem* p, int32_t shape[4]) {
    Resolved r;
    int rc = resolve(p, &r);
    if (rc != HOGATT_OK) return rc;
    if (!shape || !p->fragment_rows) return HOGATT_ERR_NULL_POINTER;
    int dev, sms, smem_optin;
    rc = current_device_info(&dev, &sms, &smem_optin);
    if (rc != HOGATT_OK) return rc;
    const int grid = grid_size(p, sms);
    refine_row_blocks(p, &r, grid, tiles_upper_bound(p, r));
    const int cluster = choose_cluster(p, r, dev, sms, smem_optin, tiles_upper_bound(p, r));
    if (r.cluster_forced && cluster == 0) return HOGATT_ERR_BAD_KERNEL_CHOICE;
    shape[0] = cluster ? HOGATT_KERNEL_MMA_CLUSTER : r.kernel;
    shape[1] = cluster ? r.units * cluster : grid;
    shape[2] = cluster;
    shape[3] = cluster ? 1 : (r.kernel == HOGATT_KERNEL_DENSE && p->cosines ? 3 : 2);
    return HOGATT_OK;
}

int hogatt_plan_ranges(int32_t tiles_per_unit, int32_t units, int32_t ctas, int32_t cta, int32_t unit, int64_t range[4]) {
    if (!range) return HOGATT_ERR_NULL_POINTER;
    if (tiles_per_unit <= 0 || units <= 0 || ctas <= 0 || cta < 0 || cta >= ctas || unit < 0 || unit >= units)
        return HOGATT_ERR_BAD_SHAPE;
    const int64_t n = (int64_t)tiles_per_unit * units;
    if (ctas > n) return HOGATT_ERR_BAD_SHAPE;
    range[0] = cta_first_tile(cta, n, ctas);
    range[1] = cta_first_tile(cta + 1, n, ctas);
    int first, count;
    unit_ctas(unit, tiles_per_unit, n, ctas, &first, &count);
    range[2] = first;
    range[3] = count;
    return HOGATT_OK;
}

}  // extern "C"
