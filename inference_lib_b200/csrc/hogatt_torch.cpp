// Thin torch binding over the C ABI of libhogatt_b200.so.
//
// Registers the operator library `libhogatt` with the schemas of the reference
// (src/binding.cu:360-386), CUDA dispatch key only, so that Python code written against
// `torch.ops.libhogatt.*` runs unchanged.  Everything here is host code: shape checks that
// mirror src/binding.cu:39-108 and :217-253, a workspace from torch's caching allocator, and one
// call into the C ABI on the current stream of the tensors' device.
#include <ATen/Tensor.h>
#include <ATen/ops/empty.h>
#include <Python.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/library.h>

#include <algorithm>
#include <vector>

#include "../../include/hogatt.h"

namespace {

int dtype_code(const at::Tensor& t) {
    if (t.scalar_type() == at::kFloat) return HOGATT_F32;
    if (t.scalar_type() == at::kHalf) return HOGATT_F16;
    if (t.scalar_type() == at::kBFloat16) return HOGATT_BF16;
    TORCH_CHECK(false, "libhogatt: unsupported dtype ", t.scalar_type(), " (float32, float16, bfloat16)");
    return -1;
}

void check_status(int rc, const char* what) {
    TORCH_CHECK(rc == HOGATT_OK, "libhogatt::", what, ": ", hogatt_status_string(rc),
                rc == HOGATT_ERR_CUDA ? " / cudaError " : "", rc == HOGATT_ERR_CUDA ? hogatt_last_cuda_error() : 0);
}

// Shared by hogwild_sdpa (rotated == true: queries [F,W,Hq,S,E]) and hogwild_fused
// (queries [W,Hq,S,E] plus cos/sin tables and the rq output).
void run_attention(at::Tensor& out, at::Tensor* rq, double scale, const at::Tensor& locations,
                   const at::Tensor& queries, const at::Tensor& fragment_lengths,
                   const std::vector<at::Tensor>& key_fragments, const std::vector<at::Tensor>& value_fragments,
                   const at::Tensor* cosines, const at::Tensor* sines, const std::vector<int64_t>* host_lengths = nullptr,
                   int64_t stable_fragments = 0) {
    const bool fused = cosines != nullptr;
    TORCH_CHECK(out.is_cuda(), "libhogatt: tensors must live on a CUDA device");
    const c10::cuda::CUDAGuard guard(out.device());
    TORCH_CHECK(out.dim() == 4 && out.is_contiguous(), "output must be contiguous [W,Hq,S,Ev]");
    const int W = out.size(0), Hq = out.size(1), S = out.size(2), Ev = out.size(3);

    TORCH_CHECK(locations.dim() == 3 && locations.is_contiguous() && locations.scalar_type() == at::kInt,
                "locations must be contiguous int32 [F,W,S]");
    const int F = locations.size(0);
    TORCH_CHECK(F > 0, "libhogatt: at least one fragment is needed");
    TORCH_CHECK_EQ(locations.size(1), W);
    TORCH_CHECK_EQ(locations.size(2), S);

    TORCH_CHECK(queries.is_contiguous() && queries.scalar_type() == out.scalar_type(), "queries: contiguous, dtype of output");
    int E;
    if (fused) {
        TORCH_CHECK(queries.dim() == 4, "queries must be [W,Hq,S,E]");
        TORCH_CHECK_EQ(queries.size(0), W);
        TORCH_CHECK_EQ(queries.size(1), Hq);
        TORCH_CHECK_EQ(queries.size(2), S);
        E = queries.size(3);
    } else {
        TORCH_CHECK(queries.dim() == 5, "queries must be [F,W,Hq,S,E]");
        TORCH_CHECK_EQ(queries.size(0), F);
        TORCH_CHECK_EQ(queries.size(1), W);
        TORCH_CHECK_EQ(queries.size(2), Hq);
        TORCH_CHECK_EQ(queries.size(3), S);
        E = queries.size(4);
    }

    TORCH_CHECK(fragment_lengths.dim() == 1 && fragment_lengths.is_contiguous() &&
                    fragment_lengths.scalar_type() == at::kInt, "fragment_lengths must be contiguous int32 [F]");
    TORCH_CHECK_EQ(fragment_lengths.size(0), F);
    TORCH_CHECK_EQ((int64_t)key_fragments.size(), (int64_t)F);
    TORCH_CHECK_EQ((int64_t)value_fragments.size(), (int64_t)F);

    for (const at::Tensor* t : {&locations, &queries, &fragment_lengths, cosines, sines, (const at::Tensor*)rq})
        TORCH_CHECK(t == nullptr || t->device() == out.device(), "libhogatt: every tensor must be on the output's device");

    std::vector<const void*> kptr(F), vptr(F);
    std::vector<int32_t> rows(F), bound(F);
    const int fo = key_fragments[0].dim() == 4 ? 1 : 0;
    const int Hkv = key_fragments[0].size(fo);
    for (int f = 0; f < F; ++f) {
        const at::Tensor& k = key_fragments[f];
        const at::Tensor& v = value_fragments[f];
        TORCH_CHECK(k.dim() == 3 + fo && v.dim() == 3 + fo, "fragments must all be [Hkv,L,E] or all [1,Hkv,L,E]");
        if (fo) TORCH_CHECK(k.size(0) == 1 && v.size(0) == 1, "the leading fragment dim must be 1");
        TORCH_CHECK_EQ(k.size(fo + 0), Hkv);
        TORCH_CHECK_EQ(v.size(fo + 0), Hkv);
        TORCH_CHECK_EQ(v.size(fo + 1), k.size(fo + 1));
        TORCH_CHECK_EQ(k.size(fo + 2), E);
        TORCH_CHECK_EQ(v.size(fo + 2), Ev);
        TORCH_CHECK(k.is_contiguous() && v.is_contiguous(), "fragments must be contiguous");
        TORCH_CHECK(k.scalar_type() == out.scalar_type() && v.scalar_type() == out.scalar_type(), "fragment dtype != output dtype");
        TORCH_CHECK(k.device() == out.device() && v.device() == out.device(), "fragments on another device");
        kptr[f] = k.const_data_ptr();
        vptr[f] = v.const_data_ptr();
        rows[f] = (int32_t)k.size(fo + 1);
        // What the host knows about the fragment's length: the reference's callers pass tensors that end at the
        // fragment's length (python/hogwild/attention.py:26-35, :160-162), so without better knowledge the row
        // count is the bound; a caller that keeps fragments in larger slabs passes its own numbers.
        bound[f] = host_lengths ? (int32_t)std::max<int64_t>(0, std::min<int64_t>((*host_lengths)[f], rows[f])) : rows[f];
    }

    hogatt_problem p = {};
    p.F = F; p.W = W; p.Hq = Hq; p.Hkv = Hkv; p.E = E; p.Ev = Ev; p.S = S;
    p.dtype = dtype_code(out);
    p.scale = (float)scale;
    p.out = out.data_ptr();
    p.queries = queries.const_data_ptr();
    p.locations = locations.const_data_ptr<int>();
    p.fragment_lengths = fragment_lengths.const_data_ptr<int>();
    p.key_fragments = kptr.data();
    p.value_fragments = vptr.data();
    p.fragment_rows = rows.data();
    p.host_lengths = bound.data();
    p.stable_fragments = (int32_t)std::max<int64_t>(0, std::min<int64_t>(stable_fragments, F));
    if (fused) {
        TORCH_CHECK(cosines->dim() == 4 && sines->dim() == 4 && cosines->is_contiguous() && sines->is_contiguous() &&
                        cosines->scalar_type() == at::kFloat && sines->scalar_type() == at::kFloat,
                    "cosines/sines must be contiguous float32 [F,W,S,R]");
        for (const at::Tensor* t : {cosines, sines}) {
            TORCH_CHECK_EQ(t->size(0), F);
            TORCH_CHECK_EQ(t->size(1), W);
            TORCH_CHECK_EQ(t->size(2), S);
        }
        TORCH_CHECK_EQ(sines->size(3), cosines->size(3));
        p.rotary_dim = (int32_t)cosines->size(3);
        p.cosines = cosines->const_data_ptr<float>();
        p.sines = sines->const_data_ptr<float>();
        if (rq != nullptr) {
            TORCH_CHECK(rq->dim() == 5 && rq->is_contiguous() && rq->scalar_type() == out.scalar_type(),
                        "rq must be contiguous [F,W,Hq,S,E]");
            TORCH_CHECK_EQ(rq->size(0), F);
            TORCH_CHECK_EQ(rq->size(1), W);
            TORCH_CHECK_EQ(rq->size(2), Hq);
            TORCH_CHECK_EQ(rq->size(3), S);
            TORCH_CHECK_EQ(rq->size(4), E);
            p.rq = rq->data_ptr();
        }
    }

    const size_t need = hogatt_workspace_bytes(&p);
    TORCH_CHECK(need > 0, "libhogatt: unsupported problem (head sizes ", E, "/", Ev, ", dtype ", out.scalar_type(), ")");
    at::Tensor workspace = at::empty({(int64_t)need}, out.options().dtype(at::kByte));
    p.workspace = workspace.data_ptr();
    p.workspace_bytes = need;

    const cudaStream_t stream = c10::cuda::getCurrentCUDAStream();
    const int rc = fused ? hogatt_fused_launch(&p, reinterpret_cast<hogatt_stream_t>(stream))
                         : hogatt_sdpa_launch(&p, reinterpret_cast<hogatt_stream_t>(stream));
    check_status(rc, fused ? "hogwild_fused" : "hogwild_sdpa");
}

// --- operators, same names and argument order as src/binding.cu:255-340 -------------------------

void hogwild_attention(at::Tensor& out, double scale, const at::Tensor& locations, const at::Tensor& queries,
                       const at::Tensor& fragment_lengths, const std::vector<at::Tensor>& key_fragments,
                       const std::vector<at::Tensor>& value_fragments) {
    run_attention(out, nullptr, scale, locations, queries, fragment_lengths, key_fragments, value_fragments, nullptr, nullptr);
}

void hogwild_rope(at::Tensor& out, const at::Tensor& queries, const at::Tensor& cosines, const at::Tensor& sines) {
    TORCH_CHECK(out.is_cuda(), "libhogatt: tensors must live on a CUDA device");
    const c10::cuda::CUDAGuard guard(out.device());
    TORCH_CHECK(out.dim() == 5 && queries.dim() == 4 && cosines.dim() == 4 && sines.dim() == 4, "hogwild_rope: bad ranks");
    TORCH_CHECK(out.is_contiguous() && queries.is_contiguous() && cosines.is_contiguous() && sines.is_contiguous());
    const int F = out.size(0), W = out.size(1), Hq = out.size(2), S = out.size(3), E = out.size(4);
    const int R = cosines.size(3);
    TORCH_CHECK_EQ(queries.size(0), W);
    TORCH_CHECK_EQ(queries.size(1), Hq);
    TORCH_CHECK_EQ(queries.size(2), S);
    TORCH_CHECK_EQ(queries.size(3), E);
    for (const at::Tensor* t : {&cosines, &sines}) {
        TORCH_CHECK(t->scalar_type() == at::kFloat, "cosines/sines must be float32");
        TORCH_CHECK_EQ(t->size(0), F);
        TORCH_CHECK_EQ(t->size(1), W);
        TORCH_CHECK_EQ(t->size(2), S);
        TORCH_CHECK_EQ(t->size(3), R);
    }
    TORCH_CHECK(queries.scalar_type() == out.scalar_type(), "queries dtype != output dtype");
    const cudaStream_t stream = c10::cuda::getCurrentCUDAStream();
    check_status(hogatt_rope_launch(out.data_ptr(), queries.const_data_ptr(), cosines.const_data_ptr<float>(),
                                    sines.const_data_ptr<float>(), F, W, Hq, S, E, R, dtype_code(out),
                                    reinterpret_cast<hogatt_stream_t>(stream)),
                 "hogwild_rope");
}

void hogwild_fused(at::Tensor& out, at::Tensor& rotated_queries, double scale, const at::Tensor& locations,
                   const at::Tensor& queries, const at::Tensor& fragment_lengths,
                   const std::vector<at::Tensor>& key_fragments, const std::vector<at::Tensor>& value_fragments,
                   const at::Tensor& cosines, const at::Tensor& sines) {
    // the reference makes every fragment contiguous here (src/binding.cu:330-337)
    std::vector<at::Tensor> keys, vals;
    keys.reserve(key_fragments.size());
    vals.reserve(value_fragments.size());
    for (size_t i = 0; i < key_fragments.size(); ++i) {
        keys.push_back(key_fragments[i].contiguous());
        vals.push_back(value_fragments[i].contiguous());
    }
    run_attention(out, &rotated_queries, scale, locations, queries, fragment_lengths, keys, vals, &cosines, &sines);
}

// hogwild_fused for callers that keep every fragment in a preallocated slab [Hkv, capacity, E] (no copies are
// made here, the slabs must be contiguous) and know on the host how long each fragment can be at most:
// `host_lengths[f]` bounds the visible rows of fragment f, `stable_fragments` leading fragments are not written
// by work enqueued before this call (see hogatt_problem in include/hogatt.h).  No counterpart in the reference.
void hogwild_fused_planned(at::Tensor& out, at::Tensor& rotated_queries, double scale, const at::Tensor& locations,
                           const at::Tensor& queries, const at::Tensor& fragment_lengths,
                           const std::vector<at::Tensor>& key_fragments, const std::vector<at::Tensor>& value_fragments,
                           const at::Tensor& cosines, const at::Tensor& sines, const std::vector<int64_t>& host_lengths,
                           int64_t stable_fragments) {
    TORCH_CHECK_EQ((int64_t)host_lengths.size(), (int64_t)key_fragments.size());
    run_attention(out, &rotated_queries, scale, locations, queries, fragment_lengths, key_fragments, value_fragments,
                  &cosines, &sines, &host_lengths, stable_fragments);
}

// --- paged operators (src/binding.cu:269-322) --------------------------------------------------------

void run_paged(at::Tensor& out, double scale, const at::Tensor& locations, const at::Tensor& queries,
               const at::Tensor& fragment_lengths, const at::Tensor& key_cache, const at::Tensor& value_cache,
               const at::Tensor& block_table, const at::Tensor* cu_seqlens_q) {
    TORCH_CHECK(out.is_cuda(), "libhogatt: tensors must live on a CUDA device");
    const c10::cuda::CUDAGuard guard(out.device());
    const bool packed = cu_seqlens_q != nullptr;
    for (const at::Tensor* t : std::initializer_list<const at::Tensor*>{&out, &locations, &queries, &fragment_lengths, &key_cache, &value_cache, &block_table})
        TORCH_CHECK(t->is_contiguous() && t->device() == out.device(), "paged attention: tensors must be contiguous and on one device");
    TORCH_CHECK(locations.scalar_type() == at::kInt && fragment_lengths.scalar_type() == at::kInt &&
                    block_table.scalar_type() == at::kInt, "locations, fragment_lengths, block_table must be int32");
    TORCH_CHECK(queries.scalar_type() == out.scalar_type() && key_cache.scalar_type() == out.scalar_type() &&
                    value_cache.scalar_type() == out.scalar_type(), "queries / caches must have the dtype of output");
    TORCH_CHECK(key_cache.dim() == 4 && value_cache.dim() == 4 && block_table.dim() == 2, "caches [NumBlocks,Hkv,bs,E], block_table [W,max_blocks]");
    hogatt_paged_problem p = {};
    p.F = (int32_t)locations.size(0);
    p.Hkv = (int32_t)key_cache.size(1);
    p.block_size = (int32_t)key_cache.size(2);
    p.max_blocks_per_seq = (int32_t)block_table.size(1);
    TORCH_CHECK_EQ(value_cache.size(1), key_cache.size(1));
    TORCH_CHECK_EQ(value_cache.size(2), key_cache.size(2));
    if (packed) {
        TORCH_CHECK(out.dim() == 3 && queries.dim() == 4 && locations.dim() == 2 && fragment_lengths.dim() == 2,
                    "varlen: out [total_q,Hq,Ev], queries [F,total_q,Hq,E], locations [F,total_q], fragment_lengths [F,W]");
        TORCH_CHECK(cu_seqlens_q->scalar_type() == at::kInt && cu_seqlens_q->is_contiguous() && cu_seqlens_q->dim() == 1);
        p.W = (int32_t)cu_seqlens_q->size(0) - 1;
        p.total_q_tokens = (int32_t)out.size(0);
        p.Hq = (int32_t)out.size(1);
        p.Ev = (int32_t)out.size(2);
        p.E = (int32_t)queries.size(3);
        TORCH_CHECK_EQ(queries.size(0), p.F);
        TORCH_CHECK_EQ(queries.size(1), p.total_q_tokens);
        TORCH_CHECK_EQ(queries.size(2), p.Hq);
        TORCH_CHECK_EQ(locations.size(1), p.total_q_tokens);
        TORCH_CHECK_EQ(fragment_lengths.size(0), p.F);
        TORCH_CHECK_EQ(fragment_lengths.size(1), p.W);
        p.cu_seqlens_q = cu_seqlens_q->const_data_ptr<int>();
    } else {
        TORCH_CHECK(out.dim() == 4 && queries.dim() == 5 && locations.dim() == 3 && fragment_lengths.dim() == 1,
                    "paged: out [W,Hq,S,Ev], queries [F,W,Hq,S,E], locations [F,W,S], fragment_lengths [F]");
        p.W = (int32_t)out.size(0);
        p.Hq = (int32_t)out.size(1);
        p.S = (int32_t)out.size(2);
        p.Ev = (int32_t)out.size(3);
        p.E = (int32_t)queries.size(4);
        TORCH_CHECK_EQ(queries.size(0), p.F);
        TORCH_CHECK_EQ(queries.size(1), p.W);
        TORCH_CHECK_EQ(queries.size(2), p.Hq);
        TORCH_CHECK_EQ(queries.size(3), p.S);
        TORCH_CHECK_EQ(locations.size(1), p.W);
        TORCH_CHECK_EQ(locations.size(2), p.S);
        TORCH_CHECK_EQ(fragment_lengths.size(0), p.F);
    }
    TORCH_CHECK_EQ(block_table.size(0), p.W);
    TORCH_CHECK_EQ(key_cache.size(3), p.E);
    TORCH_CHECK_EQ(value_cache.size(3), p.Ev);
    p.dtype = dtype_code(out);
    p.scale = (float)scale;
    p.out = out.data_ptr();
    p.queries = queries.const_data_ptr();
    p.locations = locations.const_data_ptr<int>();
    p.fragment_lengths = fragment_lengths.const_data_ptr<int>();
    p.key_cache = key_cache.const_data_ptr();
    p.value_cache = value_cache.const_data_ptr();
    p.block_table = block_table.const_data_ptr<int>();
    if (packed && p.total_q_tokens == 0) return;
    const size_t need = hogatt_paged_workspace_bytes(&p);
    TORCH_CHECK(need > 0, "libhogatt: unsupported paged problem (head sizes ", p.E, "/", p.Ev, ", Hq ", p.Hq, ", Hkv ", p.Hkv, ")");
    at::Tensor workspace = at::empty({(int64_t)need}, out.options().dtype(at::kByte));
    p.workspace = workspace.data_ptr();
    p.workspace_bytes = need;
    const cudaStream_t stream = c10::cuda::getCurrentCUDAStream();
    check_status(hogatt_paged_sdpa_launch(&p, reinterpret_cast<hogatt_stream_t>(stream)),
                 packed ? "hogwild_varlen_paged_sdpa" : "hogwild_paged_sdpa");
}

void hogwild_paged_attention(at::Tensor& out, double scale, const at::Tensor& locations, const at::Tensor& queries,
                             const at::Tensor& fragment_lengths, const at::Tensor& key_cache,
                             const at::Tensor& value_cache, const at::Tensor& block_table) {
    run_paged(out, scale, locations, queries, fragment_lengths, key_cache, value_cache, block_table, nullptr);
}

void hogwild_varlen_paged_attention(at::Tensor& out, double scale, const at::Tensor& locations, const at::Tensor& queries,
                                    const at::Tensor& fragment_lengths, const at::Tensor& key_cache,
                                    const at::Tensor& value_cache, const at::Tensor& block_table,
                                    const at::Tensor& cu_seqlens_q, const at::Tensor& cu_seqlens_k) {
    (void)cu_seqlens_k;      // carried by the reference's Shape but never read by its kernels either
    run_paged(out, scale, locations, queries, fragment_lengths, key_cache, value_cache, block_table, &cu_seqlens_q);
}

void copy_to_blocks(const at::Tensor& key_states, const at::Tensor& value_states, at::Tensor& key_cache,
                    at::Tensor& value_cache, const at::Tensor& block_table, const at::Tensor& seq_lengths) {
    TORCH_CHECK(key_states.is_cuda(), "libhogatt: tensors must live on a CUDA device");
    const c10::cuda::CUDAGuard guard(key_states.device());
    for (const at::Tensor* t : {&key_states, &value_states, &block_table, &seq_lengths})
        TORCH_CHECK(t->is_contiguous(), "copy_to_blocks: inputs must be contiguous");
    TORCH_CHECK(key_cache.is_contiguous() && value_cache.is_contiguous(), "copy_to_blocks: caches must be contiguous");
    TORCH_CHECK(key_states.dim() == 4 && value_states.dim() == 4 && key_cache.dim() == 4 && value_cache.dim() == 4 &&
                    block_table.dim() == 2 && seq_lengths.dim() == 1, "copy_to_blocks: bad ranks");
    TORCH_CHECK(block_table.scalar_type() == at::kInt && seq_lengths.scalar_type() == at::kInt, "block_table / seq_lengths must be int32");
    TORCH_CHECK(value_states.scalar_type() == key_states.scalar_type() && key_cache.scalar_type() == key_states.scalar_type() &&
                    value_cache.scalar_type() == key_states.scalar_type(), "copy_to_blocks: dtype mismatch");
    const int B = key_states.size(0), Hkv = key_states.size(1), S_new = key_states.size(2), E = key_states.size(3);
    const int Ev = value_states.size(3);
    TORCH_CHECK_EQ(value_states.size(0), B);
    TORCH_CHECK_EQ(value_states.size(1), Hkv);
    TORCH_CHECK_EQ(value_states.size(2), S_new);
    TORCH_CHECK_EQ(key_cache.size(1), Hkv);
    TORCH_CHECK_EQ(key_cache.size(3), E);
    TORCH_CHECK_EQ(value_cache.size(1), Hkv);
    TORCH_CHECK_EQ(value_cache.size(3), Ev);
    TORCH_CHECK_EQ(value_cache.size(2), key_cache.size(2));
    TORCH_CHECK_EQ(block_table.size(0), B);
    TORCH_CHECK_EQ(seq_lengths.size(0), B);
    const cudaStream_t stream = c10::cuda::getCurrentCUDAStream();
    check_status(hogatt_copy_to_blocks_launch(key_states.const_data_ptr(), value_states.const_data_ptr(), key_cache.data_ptr(),
                                              value_cache.data_ptr(), block_table.const_data_ptr<int>(),
                                              seq_lengths.const_data_ptr<int>(), B, Hkv, S_new, E, Ev, (int)key_cache.size(2),
                                              (int)block_table.size(1), dtype_code(key_states),
                                              reinterpret_cast<hogatt_stream_t>(stream)),
                 "copy_to_blocks");
}

}  // namespace

extern "C" {
// Lets the shared object be imported as an (empty) Python module, which runs the static
// registrations below -- same device as the reference's PyInit_libhogatt (src/binding.cu:342-358).
PyObject* PyInit_libhogatt(void) {
    static struct PyModuleDef module_def = {PyModuleDef_HEAD_INIT, "libhogatt", NULL, -1, NULL};
    return PyModule_Create(&module_def);
}
}

TORCH_LIBRARY(libhogatt, m) {
    std::vector<at::Tag> tags;
    tags.push_back(at::Tag::needs_fixed_stride_order);
    m.def("hogwild_sdpa(Tensor(a!) output, float scale, Tensor locations, Tensor queries, "
          "Tensor fragment_lengths, Tensor[] key_fragments, Tensor[] value_fragments) -> ()", tags, torch::_RegisterOrVerify::REGISTER);
    m.def("hogwild_rope(Tensor(a!) output, Tensor queries, Tensor cosines, Tensor sines) -> ()", tags, torch::_RegisterOrVerify::REGISTER);
    m.def("hogwild_fused(Tensor(a!) output, Tensor(b!) rq, float scale, Tensor locations, Tensor queries, "
          "Tensor fragment_lengths, Tensor[] key_fragments, Tensor[] value_fragments, Tensor cosines, Tensor sines) -> ()", tags, torch::_RegisterOrVerify::REGISTER);
    m.def("hogwild_paged_sdpa(Tensor(a!) output, float scale, Tensor locations, Tensor queries, "
          "Tensor fragment_lengths, Tensor key_cache, Tensor value_cache, Tensor block_table) -> ()", tags, torch::_RegisterOrVerify::REGISTER);
    m.def("copy_to_blocks(Tensor key_states, Tensor value_states, Tensor(a!) key_cache, Tensor(b!) value_cache, "
          "Tensor block_table, Tensor seq_lengths) -> ()", tags, torch::_RegisterOrVerify::REGISTER);
    m.def("hogwild_varlen_paged_sdpa(Tensor(a!) output, float scale, Tensor locations, Tensor queries, "
          "Tensor fragment_lengths, Tensor key_cache, Tensor value_cache, Tensor block_table, Tensor cu_seqlens_q, Tensor cu_seqlens_k) -> ()", tags, torch::_RegisterOrVerify::REGISTER);
    // beyond the reference's six operators: hogwild_fused with the host's knowledge of the fragment lengths
    m.def("hogwild_fused_planned(Tensor(a!) output, Tensor(b!) rq, float scale, Tensor locations, Tensor queries, "
          "Tensor fragment_lengths, Tensor[] key_fragments, Tensor[] value_fragments, Tensor cosines, Tensor sines, "
          "int[] host_lengths, int stable_fragments) -> ()", tags, torch::_RegisterOrVerify::REGISTER);
}

TORCH_LIBRARY_IMPL(libhogatt, CUDA, m) {
    m.impl("hogwild_sdpa", hogwild_attention);
    m.impl("hogwild_rope", hogwild_rope);
    m.impl("hogwild_fused", hogwild_fused);
    m.impl("hogwild_paged_sdpa", hogwild_paged_attention);
    m.impl("copy_to_blocks", copy_to_blocks);
    m.impl("hogwild_varlen_paged_sdpa", hogwild_varlen_paged_attention);
    m.impl("hogwild_fused_planned", hogwild_fused_planned);
}
