/*
 * hogatt.h -- C ABI of the B200-native Hogwild! fragmented-KV attention library
 * (libhogatt_b200.so).
 *
 * The reference project has no C ABI of its own: its torch operators (src/binding.cu:360-386)
 * call C++ templates (src/kernels/kernel_v21.cuh:951-1086, src/rope.cuh:54-62) with raw pointers
 * and a `Shape` POD (src/common.h:5-20).  The functions below are that same layer, cut at the
 * raw-pointer level, so that a binding in any language can replace the reference launchers one
 * for one.  Each entry point names the reference interface it stands in for.
 *
 * Conventions
 *   - Plain C types only.  Every pointer marked "device" must be dereferenceable by the GPU that is
 *     current on the calling thread; every pointer marked "host" is read during the call only.
 *   - All tensors are dense and row-major in the stated shape (the reference checks
 *     `is_contiguous()` on each of them, src/binding.cu:51-97).  Key/value rows and query rows must
 *     start on a 16-byte boundary (the reference's 16-byte vector loads need the same).
 *   - Nothing here allocates, frees or synchronises (except where an entry point says otherwise):
 *     scratch memory comes from the caller (`hogatt_workspace_bytes`), work is enqueued on the
 *     stream given, and the call returns as soon as the launches are queued.  Calls are
 *     re-entrant and may be captured into a CUDA graph.
 *   - Return value: 0 on success, a negative `hogatt_status` otherwise; nothing is launched when
 *     an error is returned.  Unsupported shapes are an error (the reference prints a message and
 *     reports success with the output untouched, src/kernels/kernel_v21.cuh:992-995).
 *   - A row that can see no key at all produces zeros (as the reference kernel does,
 *     src/kernels/kernel_v21.cuh:238-245).
 */
#ifndef HOGATT_H_
#define HOGATT_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define HOGATT_ABI_VERSION 2
#ifndef HOGATT_MAX_FRAGMENTS
#define HOGATT_MAX_FRAGMENTS 128   /* the fragment table travels by value in the kernel arguments (24 bytes per
                                      fragment); the reference's device pointer table admits 512
                                      (src/binding.cu:79-82).  More fragments: HOGATT_ERR_TOO_MANY_FRAGMENTS */
#endif
#define HOGATT_MAX_PEERS 8         /* GPUs of one node that can share a gathered output */

typedef struct CUstream_st* hogatt_stream_t;   /* == cudaStream_t */

typedef enum hogatt_dtype {
    HOGATT_F32 = 0,
    HOGATT_F16 = 1,
    HOGATT_BF16 = 2
} hogatt_dtype;

typedef enum hogatt_status {
    HOGATT_OK = 0,
    HOGATT_ERR_NULL_POINTER = -1,
    HOGATT_ERR_BAD_SHAPE = -2,          /* non-positive dims, Hq not a multiple of Hkv, rotary_dim odd or > E */
    HOGATT_ERR_UNSUPPORTED_HEAD_DIM = -3,
    HOGATT_ERR_UNSUPPORTED_DTYPE = -4,
    HOGATT_ERR_TOO_MANY_FRAGMENTS = -5,
    HOGATT_ERR_MISALIGNED = -6,
    HOGATT_ERR_WORKSPACE_TOO_SMALL = -7,
    HOGATT_ERR_CUDA = -8,               /* a CUDA runtime call failed; see hogatt_last_cuda_error() */
    HOGATT_ERR_BAD_KERNEL_CHOICE = -9,
    HOGATT_ERR_TOO_LARGE = -10,
    HOGATT_ERR_EXCEEDS_STATIC_SCRATCH = -11  /* hogatt_fused_launch_static: needs more than HOGATT_STATIC_SCRATCH_BYTES */
} hogatt_status;

/* Which device code runs.  AUTO picks the tensor-core kernel for f16/bf16 with E == Ev in {64, 128}
 * and the FMA kernel for everything else (fp32, other head sizes).  The tensor-core kernel has two
 * launch shapes: a persistent grid (one CTA per SM over balanced tile ranges -- or fewer CTAs of one
 * common whole number of tiles each, where that keeps every range inside one fragment -- partial results
 * in the workspace, a merge kernel after it) and a thread-block-cluster grid (one cluster per kv head and row
 * block, partial results merged through distributed shared memory inside the same kernel, nothing
 * written to the workspace).  AUTO and MMA take the persistent grid (on B200 it is the faster one at every
 * measured shape, its merge step folding any number of partials per row in one memory round trip);
 * MMA_CLUSTER forces the cluster shape (HOGATT_ERR_BAD_KERNEL_CHOICE when there are more units than half
 * the SMs, or the device cannot hold one cluster per unit at once).  hogatt_launch_shape() tells which one
 * a problem gets.  A CTA keeps 16, 32 or 64 query rows of a kv head: normally the smallest block that holds
 * all W x Hq/Hkv x S of them (every key is then fetched once), smaller blocks for short calls with few kv
 * heads, where they are faster (hogatt_plan_describe reports the outcome).
 *
 * DENSE is the kernel for calls with many query rows per kv head (W x Hq/Hkv x S >= 128, e.g. workers that
 * each issue a 16-token chunk), where the op is bound by the tensor pipe, not by HBM: 128-row query blocks,
 * tcgen05.mma with accumulators in tensor memory, K / V / Q tiles fetched by tensor-map TMA.  f16 / bf16,
 * E == Ev == 128, at most 16 fragments, and Hq/Hkv x S must divide 128 or be a multiple of it; AUTO takes it
 * whenever a problem qualifies, DENSE forces it (HOGATT_ERR_BAD_KERNEL_CHOICE otherwise).  It reads rotated
 * queries from memory, so the fused entry point first runs the stand-alone rotation kernel into `rq` (or into
 * the workspace when rq is NULL): three kernels per call. */
typedef enum hogatt_kernel_choice {
    HOGATT_KERNEL_AUTO = 0,
    HOGATT_KERNEL_FMA = 1,
    HOGATT_KERNEL_MMA = 2,
    HOGATT_KERNEL_MMA_CLUSTER = 3,
    HOGATT_KERNEL_DENSE = 4
} hogatt_kernel_choice;

/*
 * One call of the fragment attention op.  Field names follow the reference's `Shape`
 * (src/common.h:5-20) and operator arguments (src/binding.cu:363-367).
 */
typedef struct hogatt_problem {
    int32_t F;            /* fragments                       */
    int32_t W;            /* workers                         */
    int32_t Hq;           /* query heads                     */
    int32_t Hkv;          /* key/value heads, Hq % Hkv == 0  */
    int32_t E;            /* qk head size                    */
    int32_t Ev;           /* v head size                     */
    int32_t S;            /* query tokens per worker         */
    int32_t rotary_dim;   /* R: leading channels that are rotated (ignored when cosines == NULL) */
    int32_t dtype;        /* hogatt_dtype of out, rq, queries, keys, values */
    float   scale;        /* softmax scale applied to q.k    */

    void*        out;      /* device [W,Hq,S,Ev]                                              */
    void*        rq;       /* device [F,W,Hq,S,E] or NULL: rotated queries, written when given */
    const void*  queries;  /* device: [W,Hq,S,E] un-rotated when cosines != NULL,
                                      [F,W,Hq,S,E] already rotated when cosines == NULL        */
    const float* cosines;  /* device [F,W,S,R] fp32 or NULL                                   */
    const float* sines;    /* device [F,W,S,R] fp32 or NULL                                   */
    const int32_t* locations;         /* device [F,W,S]: key l of fragment f is visible to (w,s)
                                         iff l <= locations[f,w,s]                            */
    const int32_t* fragment_lengths;  /* device [F] or NULL: visible length of each fragment;
                                         NULL means fragment_rows[f]                          */

    const void* const* key_fragments;    /* host array of F device pointers, each [Hkv, rows_f, E]  */
    const void* const* value_fragments;  /* host array of F device pointers, each [Hkv, rows_f, Ev] */
    const int32_t*     fragment_rows;    /* host array of F ints: rows_f, the token extent of the
                                            tensors (their head stride is rows_f * E)           */

    void*   workspace;        /* device scratch, >= hogatt_workspace_bytes() bytes, 256-byte aligned */
    size_t  workspace_bytes;
    int32_t* device_status;   /* device int or NULL: kernels OR a nonzero code into it when a bounded
                                 wait inside a kernel gives up (never expected in normal operation) */
    int32_t kernel;           /* hogatt_kernel_choice */
    int32_t max_ctas;         /* 0 = one CTA per SM; otherwise caps the persistent grid (testing)   */

    /* Optional knowledge the host has about this call; both may stay 0 / NULL.
     *
     * host_lengths (host array of F ints, or NULL): for every fragment an UPPER BOUND, known on the
     *   host, of the number of leading rows any query can see (the reference's callers hold exactly
     *   this number: their fragment tensors end at the fragment's length, python/hogwild/attention.py:
     *   26-35).  Values are clamped to [0, fragment_rows[f]].  When given, the tensor-core kernel cuts
     *   the call into tiles from these numbers alone, so a CTA starts streaming keys and values
     *   without first reading `locations` / `fragment_lengths` from device memory; visibility itself
     *   is still decided on the device, row by row, from `locations` and `fragment_lengths`, so rows
     *   between the true length and the bound are fetched and masked (their contents never reach a
     *   result, whatever they hold).  NULL: the tiles are derived on the device from `locations` and
     *   `fragment_lengths` (exact; one dependent memory round trip at the start of every CTA).
     *
     * stable_fragments: the keys and values of fragments 0 .. stable_fragments-1 were complete before
     *   the stream's last few kernels were enqueued and nothing enqueued since writes them (the shared
     *   prompt of a decode step, as opposed to the workers' fragments that the step has just appended
     *   to).  With host_lengths given and programmatic dependent launch in use (the default; the
     *   environment variable HOGATT_PDL=0 turns it off), the
     *   kernel fetches its first tiles of those fragments BEFORE it waits for the stream's preceding
     *   kernel, i.e. while that kernel -- and, if that kernel itself was allowed to start early, the
     *   one before it -- may still be running; after one of this library's calls that is that call's
     *   own two kernels and nothing older.  Everything else -- queries, tables, locations, lengths,
     *   the other fragments, every store -- is touched only after the wait.  0: nothing is read early. */
    const int32_t* host_lengths;
    int32_t stable_fragments;
    int32_t reserved_;
} hogatt_problem;

/* ABI version compiled into the library (== HOGATT_ABI_VERSION of the header it was built from). */
int hogatt_abi_version(void);

/* Static text for a hogatt_status. */
const char* hogatt_status_string(int status);

/* The last cudaError_t seen by this thread inside the library (0 if none), for HOGATT_ERR_CUDA. */
int hogatt_last_cuda_error(void);

/*
 * Scratch bytes hogatt_sdpa_launch / hogatt_fused_launch need for this problem on the current
 * device (split-K partial sums and their softmax statistics).  Only the dims, dtype, kernel and
 * max_ctas fields are read; the figure covers every launch shape a launch with these fields may
 * pick.  Returns 0 for an invalid problem.
 * Stands in for the grow-only static workspace of src/kernels/kernel_v21.cuh:969-980.
 */
size_t hogatt_workspace_bytes(const hogatt_problem* p);

/*
 * Attention over fragments with queries that are already rotated: problem.queries is
 * [F,W,Hq,S,E], cosines/sines/rq must be NULL.
 * Replaces v21::hogwild_attention_gpu (src/kernels/kernel_v21.cuh:951-996) as called from the
 * `hogwild_sdpa` operator (src/binding.cu:39-108,255-267).
 */
int hogatt_sdpa_launch(const hogatt_problem* p, hogatt_stream_t stream);

/*
 * Query RoPE per fragment fused into the attention prologue: problem.queries is [W,Hq,S,E],
 * cosines/sines are given; when rq != NULL the rotated queries are also written out.
 * Replaces the composition rope_gpu + v21::hogwild_attention_gpu of the `hogwild_fused` operator
 * (src/binding.cu:324-340).
 */
int hogatt_fused_launch(const hogatt_problem* p, hogatt_stream_t stream);

/*
 * hogatt_fused_launch for callers that cannot hand over scratch memory.  It has no counterpart in
 * the reference.
 *
 * Some hosts of this library are not allowed to allocate device memory at the point where they call
 * it: a plugin that runs inside another runtime's host callback, a process whose device memory is
 * owned and budgeted by a separate allocator it cannot reach from C, or a real-time loop where
 * cudaMalloc's implicit device synchronisation is forbidden.  For them the split-K partial sums live in ONE fixed array inside the library image
 * (HOGATT_STATIC_SCRATCH_BYTES of device memory on every GPU that loads the library, held until the
 * process exits) instead of `workspace`; `workspace` and `workspace_bytes` are ignored, everything
 * else is as for hogatt_fused_launch and the results are identical.
 *
 *   - A problem whose scratch need (hogatt_workspace_bytes) exceeds HOGATT_STATIC_SCRATCH_BYTES is
 *     refused with HOGATT_ERR_EXCEEDS_STATIC_SCRATCH and nothing is launched.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with
 *     that device current); make that first call outside any stream capture.  Later calls only
 *     enqueue kernels.  No call allocates or frees memory.
 *   - All calls on a device share the one array, which keeps whatever the last call left in it.
 *     Nothing has to be cleared between calls: every partial slot that enters a result was written
 *     by this call's attention kernel first.  The merge step does load slots this call did not
 *     write (it reads a fixed number per row so that the loads are in flight together) and discards
 *     them by the unit's slot count before any arithmetic, so stale bytes, NaN patterns included,
 *     never reach an output.  Two calls that overlap on the GPU (issued on different streams) race
 *     on the array: serialise them, or give the overlapping ones their own workspace through
 *     hogatt_fused_launch.
 */
#define HOGATT_STATIC_SCRATCH_BYTES (8u << 20)
int hogatt_fused_launch_static(const hogatt_problem* p, hogatt_stream_t stream);

/*
 * KV-head sharding across the GPUs of one node with the output all-gather fused into the op.
 * No counterpart in the reference (single device, src/kernels/kernel_v21.cuh:960).
 *
 * Every rank calls this with ITS shard as the problem (Hkv/world kv heads, Hq/world query heads; `out` is
 * ignored) and a table of peer-mapped pointers.  The merge step stores each finished output row straight
 * into the full-size output [W, world*Hq, S, Ev] of EVERY rank (plain stores over NVLink through the peer
 * mapping) at this rank's head offset; a one-warp kernel then publishes a per-call count to every peer
 * (release at system scope) and waits, for at most about a second (then: bit 32 in device_status;
 * HOGATT_WAIT_LIMIT_MS in the environment shortens it), until all peers have published theirs.  When the
 * call's work has completed on a rank's stream, that rank's out_full is complete.
 *   out_full[p], flags[p]: rank p's buffers as mapped into THIS GPU's address space (CUDA IPC / VMM /
 *       symmetric memory); out_full[p] is 16-byte aligned (HOGATT_ERR_MISALIGNED otherwise);
 *       flags[p] is int32[world + 1], zero-filled once before the first call
 *       (slots 0 .. world-1: the counts the ranks publish; slot world: rank p's own call counter).
 *   The caller must not let a rank start call k+1 on an out_full that another rank is still reading
 *   from call k (alternate two buffers, or synchronise the consumers).
 */
typedef struct hogatt_peers {
    int32_t  world, rank;
    void*    out_full[HOGATT_MAX_PEERS];
    int32_t* flags[HOGATT_MAX_PEERS];
} hogatt_peers;
int hogatt_fused_launch_gather(const hogatt_problem* p, const hogatt_peers* peers, hogatt_stream_t stream);

/*
 * rq[f,w,h,s,:] = rope(queries[w,h,s,:], cosines[f,w,s,:], sines[f,w,s,:]) with the rotate-half
 * pairing, channels >= R copied.  All pointers device.
 * Replaces rope_gpu (src/rope.cuh:54-62) of the `hogwild_rope` operator (src/binding.cu:217-253).
 */
int hogatt_rope_launch(void* rq, const void* queries, const float* cosines, const float* sines,
                       int32_t F, int32_t W, int32_t Hq, int32_t S, int32_t E, int32_t rotary_dim,
                       int32_t dtype, hogatt_stream_t stream);

/*
 * The paged variants.  Worker w's keys/values are one paged sequence: key l lives in block
 * block_table[w, l / block_size] at row l % block_size of cache[num_blocks, Hkv, block_size, E].
 * Every fragment index f reads that same sequence with its own (already rotated) query, location
 * and length -- the addressing of the reference kernels (src/kernels/kernel_v21.cuh:402-411).
 *   fixed layout  (cu_seqlens_q == NULL): queries [F,W,Hq,S,E], out [W,Hq,S,Ev], locations [F,W,S],
 *                 fragment_lengths [F]                       -- `hogwild_paged_sdpa`
 *   packed layout (cu_seqlens_q != NULL): queries [F,total_q,Hq,E], out [total_q,Hq,Ev],
 *                 locations [F,total_q], fragment_lengths [F,W], cu_seqlens_q [W+1] (device)
 *                                                            -- `hogwild_varlen_paged_sdpa`
 * All pointers device.  CUDA-core kernel: any of the three dtypes, E <= 256, Ev in {32,64,128,256}.
 */
typedef struct hogatt_paged_problem {
    int32_t F, W, Hq, Hkv, E, Ev;
    int32_t S;                     /* fixed layout only */
    int32_t total_q_tokens;        /* packed layout only */
    int32_t block_size, max_blocks_per_seq;
    int32_t dtype;
    float   scale;
    void*          out;
    const void*    queries;
    const int32_t* locations;
    const int32_t* fragment_lengths;
    const void*    key_cache;
    const void*    value_cache;
    const int32_t* block_table;    /* [W, max_blocks_per_seq] */
    const int32_t* cu_seqlens_q;   /* [W+1] or NULL */
    void*   workspace;             /* >= hogatt_paged_workspace_bytes(), 256-byte aligned */
    size_t  workspace_bytes;
    int32_t kernel;                /* HOGATT_KERNEL_AUTO, _FMA (CUDA cores: any dtype and head size above) or _MMA
                                      (mma.sync tensor cores: f16 / bf16 with E == Ev == 64 or 128; what AUTO takes
                                      there unless HOGATT_PAGED_MMA=0 is set in the environment) */
    int32_t reserved_;
} hogatt_paged_problem;

size_t hogatt_paged_workspace_bytes(const hogatt_paged_problem* p);

/*
 * Replaces v21::hogwild_paged_attention_gpu (src/kernels/kernel_v21.cuh:998-1043, operator
 * `hogwild_paged_sdpa`, src/binding.cu:110-142) and v21::hogwild_varlen_paged_attention_gpu
 * (:1045-1086, operator `hogwild_varlen_paged_sdpa`, src/binding.cu:144-181).
 */
int hogatt_paged_sdpa_launch(const hogatt_paged_problem* p, hogatt_stream_t stream);

/*
 * Append S_new new key/value rows per (batch, kv head) to the paged caches at positions
 * seq_lengths[b] + t.  key_states [B,Hkv,S_new,E], value_states [B,Hkv,S_new,Ev], caches
 * [num_blocks,Hkv,block_size,E/Ev], block_table [B,max_blocks], seq_lengths [B]; all device.
 * Replaces copy_to_blocks_kernel (src/cache.cuh:6-49, operator `copy_to_blocks`, src/binding.cu:183-215).
 */
int hogatt_copy_to_blocks_launch(const void* key_states, const void* value_states, void* key_cache, void* value_cache,
                                 const int32_t* block_table, const int32_t* seq_lengths, int32_t B, int32_t Hkv,
                                 int32_t S_new, int32_t E, int32_t Ev, int32_t block_size, int32_t max_blocks,
                                 int32_t dtype, hogatt_stream_t stream);

/* ---- the steps either side of the attention op in a decode step ------------------------------------- */

/*
 * Per-step metadata, on the device.  Every worker sees the same F fragments, each in its own order
 * (shared prompt first, other workers' fragments, its own last); a new token's position with respect
 * to fragment f is counted from the END of the worker's sequence: the fragment that comes last in the
 * order ends at its own length, the one before it at the sum of both lengths, and so on, and token s
 * of the S new ones sits at end - S + s.  Writes locations[f,w,s] (what hogatt_problem.locations takes)
 * and the rotary tables for those positions, cos/sin[f,w,s,:] = cos/sin(position * inv_freq[i]) *
 * attention_scaling with both halves equal (what hogatt_problem.cosines / sines take).
 * A fragment that is missing from a worker's order gets location -1 (nothing visible).
 * Replaces the layer-0 block of HogwildCache.update (python/hogwild/attention.py:164-204): Python loops
 * over workers and fragments, torch.stack, and the model's rotary_emb, on every step.
 */
typedef struct hogatt_step_plan {
    int32_t F, W, S, rotary_dim;
    const int32_t* order;             /* device [W][F]: fragment ids in worker w's order, -1 after the last */
    const int32_t* fragment_lengths;  /* device [F]: lengths INCLUDING the S tokens of this step            */
    const float*   inv_freq;          /* device [rotary_dim / 2]                                            */
    float   attention_scaling;        /* 1.0 for plain RoPE                                                 */
    int32_t round_tables_to;          /* hogatt_dtype: HOGATT_F32 keeps the fp32 values; F16 / BF16 rounds
                                         them to that type first, as rotary_emb does when it returns tables
                                         in the model's type and the reference converts them back to float
                                         (attention.py:191-193)                                             */
    int32_t* locations;               /* out, device [F,W,S]                                                */
    float*   cosines;                 /* out, device [F,W,S,rotary_dim] fp32                                */
    float*   sines;
} hogatt_step_plan;

int hogatt_step_plan_launch(const hogatt_step_plan* p, hogatt_stream_t stream);

/*
 * K-side write path: rotate the new keys of every source at their own positions and append keys and
 * values to the source's destination fragment, in place.  Fragments are preallocated slabs
 * [Hkv, fragment_rows[f], E]: their pointers never change, the lengths live on the device.  Source w
 * contributes its last (take_leading: first) new_rows[w] rows (all S when new_rows is NULL) at rows
 * lengths_in[f] ... of fragment f = write_to[w]; sources that share a fragment follow each other in
 * source order.  lengths_out[f] = lengths_in[f] + rows appended (a DIFFERENT buffer than lengths_in).
 * Rows that do not fit into the slab are dropped and 256 is ORed into *device_status.
 *   - table_dtype == HOGATT_F32: fp32 tables, products in fp32, one rounding to the tensors' type
 *     (the arithmetic of hogwild_rope on queries);
 *   - table_dtype == dtype: tables in the tensors' type, each product and the sum rounded to it -- what
 *     torch computes in AttentionModule.forward, apply_rotary_pos_emb(key_states, cos, sin) with the
 *     model's position_embeddings (python/hogwild/attention.py:84-90, :315).
 * Replaces that call together with HogwildCache.update's write_to[w].update(...) (attention.py:148-158,
 * a torch.cat per worker and layer) and, with one source whose table row is broadcast
 * (table_strides = {0, 0}), the re-rotation loop of merge_caches (attention.py:251-257).
 */
#define HOGATT_MAX_APPEND_SOURCES 64
typedef struct hogatt_append {
    int32_t W, Hkv, E, Ev, S, rotary_dim, dtype, table_dtype;
    const void* keys;              /* device; element (w, h, s, e) at keys + w*ks[0] + h*ks[1] + s*ks[2] + e   */
    int64_t     key_strides[3];
    const void* values;
    int64_t     value_strides[3];
    const void* cosines;           /* device; row (w, s) at cosines + w*ts[0] + s*ts[1], rotary_dim entries    */
    const void* sines;
    int64_t     table_strides[2];
    const int32_t* new_rows;       /* device [W] or NULL                                                       */
    const int32_t* write_to;       /* host [W]: destination fragment of every source                           */
    int32_t F;
    int32_t take_leading;          /* 0: new_rows counts from the END of a source (left-masked model input);
                                      1: from its START (the source is itself a slab with new_rows valid rows,
                                      as in merge_caches)                                                      */
    void* const* key_fragments;    /* host array of F device pointers, [Hkv, fragment_rows[f], E]              */
    void* const* value_fragments;  /* host array of F device pointers, [Hkv, fragment_rows[f], Ev]             */
    const int32_t* fragment_rows;  /* host [F]: capacity of each slab in rows                                  */
    const int32_t* lengths_in;     /* device [F]                                                               */
    int32_t*       lengths_out;    /* device [F], not the same buffer as lengths_in                            */
    int32_t*       device_status;  /* device int or NULL                                                       */
} hogatt_append;

int hogatt_append_launch(const hogatt_append* p, hogatt_stream_t stream);

/*
 * Host-only description of how a problem is cut into work for the persistent grid; no GPU needed.
 * `visible_rows[f]` is the number of leading keys of fragment f that some query row can see.
 * Fills: plan[0] = tokens per tile, plan[1] = rows per row block, plan[2] = row blocks,
 * plan[3] = tiles per (row block, kv head) unit, plan[4] = units, plan[5] = CTAs that get work
 * (cluster shape: units x CTAs per cluster), plan[6] = partial-result slots per unit (cluster shape:
 * CTAs per cluster), plan[7] = kernel chosen (hogatt_kernel_choice; HOGATT_KERNEL_MMA_CLUSTER when
 * the cluster shape would run, taking visible_rows as the fragments' row counts).
 * Used by the tests of the split-K decomposition; has no reference counterpart (the reference
 * derives `splits` inline, src/kernels/kernel_v21.cuh:957-964).
 */
int hogatt_plan_describe(const hogatt_problem* p, const int32_t* visible_rows, int32_t num_sms,
                         int32_t plan[8]);

/*
 * What one hogatt_sdpa_launch / hogatt_fused_launch of this problem enqueues on the current device
 * (dims, dtype, kernel, max_ctas and fragment_rows are read): shape[0] = device code
 * (hogatt_kernel_choice, never AUTO), shape[1] = CTAs of the attention grid, shape[2] = CTAs per
 * cluster (0: no clusters; an upper bound, a forced cluster launch shrinks it until all clusters are
 * resident), shape[3] = kernels per call (1 when the attention kernel merges by itself, 2 with the
 * merge kernel).  No reference counterpart.
 */
int hogatt_launch_shape(const hogatt_problem* p, int32_t shape[4]);

/*
 * For the decomposition above: the half-open range of global tile indices CTA `cta` walks
 * (range[0], range[1]) and, for unit `unit`, the first CTA that touches it and how many do
 * (range[2], range[3]).  Host-only.
 */
int hogatt_plan_ranges(int32_t tiles_per_unit, int32_t units, int32_t ctas, int32_t cta, int32_t unit,
                       int64_t range[4]);

#ifdef __cplusplus
}
#endif
#endif /* HOGATT_H_ */
