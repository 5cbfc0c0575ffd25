// Torch extension module `decoding_attn_cuda`: the call surface of the reference's binding
// (csrc/torch/decoding_torch.cpp:19-85) on top of this library's C ABI.
//
//   fwd(q, k, v_, o_, cu_seq_k, max_seq_k, dim_v, is_alibi) -> o      same positional signature and
//       checks as the reference's dmha_fwd (decoding_torch.cpp:19-80); v_ = None selects MLA.
//   dmha_fwd(q, k, v, cu_seq_k, max_seq_k, is_alibi, softmax_scale=None, out=None, return_lse=False, k_scale=1, v_scale=1)
//       (k, v may be torch.float8_e4m3fn: an FP8 cache standing for k * k_scale, v * v_scale)
//   dmla_fwd(q, kv, cu_seq_k, max_seq_k, dim_v=512, is_alibi=False, softmax_scale=None, out=None, return_lse=False)
//       the two named entry points with an explicit softmax scale; their defaults reproduce fwd().
//   merge_partials(part_o, part_lse, out_dtype) -> (o, lse)           LSE merge of key-range shards.
//
// Differences from the reference, all on the safe side: a device guard on q's device (the
// reference takes none, so it only works on the current device), real row strides are passed down
// instead of assuming packed rows (decoding_attn.cpp:32-46), and library errors raise instead of
// terminating the process.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <cstring>
#include <optional>
#include <tuple>

#include "../../include/decoding_attn_b200.h"

namespace {

#define DA_CHECK_DEVICE(x) TORCH_CHECK(x.is_cuda(), #x " must be on CUDA")
#define DA_CHECK_SHAPE(x, ...) \
    TORCH_CHECK(x.sizes() == torch::IntArrayRef({__VA_ARGS__}), #x " must have shape (" #__VA_ARGS__ ")")
#define DA_CHECK_CONTIGUOUS(x) TORCH_CHECK(x.is_contiguous(), #x " must be contiguous")

struct Outputs {
    at::Tensor o;
    at::Tensor lse;
};

Outputs run(const at::Tensor &q, const at::Tensor &k, const std::optional<at::Tensor> &v_,
            const std::optional<at::Tensor> &o_, const at::Tensor &cu_seq_k, int64_t max_seq_k, int64_t dim_v,
            bool is_alibi, std::optional<double> softmax_scale, bool want_lse, const at::Tensor *block_table = nullptr,
            int64_t page_size = 0, double k_scale = 1.0, double v_scale = 1.0) {
    auto q_dtype = q.dtype();
    TORCH_CHECK(q_dtype == torch::kFloat16 || q_dtype == torch::kBFloat16,
                "Decoding-Attention only support FP16 and BF16 data type");
    const bool is_bf16 = q_dtype == torch::kBFloat16;
    // An FP8 e4m3 cache (k and v both) is an extension; the reference requires the dtype of q
    // (csrc/torch/decoding_torch.cpp:28, :57).
    // A quantised cache (k and v both) is an extension: FP8 e4m3, or int8 (torch.int8); int4 goes through the C ABI.
    const bool int8_cache = k.scalar_type() == at::kChar;
    const bool fp8_cache = k.scalar_type() == at::kFloat8_e4m3fn || int8_cache;
    TORCH_CHECK(fp8_cache || k.dtype() == q_dtype, "query and key must have the same dtype");
    TORCH_CHECK(cu_seq_k.dtype() == torch::kInt32, "cu_seq_k must have dtype int32");

    DA_CHECK_DEVICE(q);
    DA_CHECK_DEVICE(k);
    DA_CHECK_DEVICE(cu_seq_k);
    TORCH_CHECK(k.device() == q.device() && cu_seq_k.device() == q.device(), "all tensors must be on one device");
    TORCH_CHECK(q.dim() == 3 && k.dim() == 3, "query and key must be 3-D");

    TORCH_CHECK(q.stride(-1) == 1, "query must have contiguous last dimension");
    TORCH_CHECK(k.stride(-1) == 1, "key must have contiguous last dimension");
    DA_CHECK_CONTIGUOUS(cu_seq_k);

    const int64_t batch = cu_seq_k.numel() - 1;
    const int64_t total_q = q.size(0);
    const int64_t head_q = q.size(1);
    const int64_t dim = q.size(2);
    const int64_t total_k = k.size(0);
    const int64_t head_k = k.size(1);
    TORCH_CHECK(batch > 0, "batch size must be positive");
    TORCH_CHECK(total_q == batch, "one query token per sequence: q.size(0) must equal cu_seq_k.numel() - 1");
    TORCH_CHECK(dim <= 576, "dim should be at most 576");
    TORCH_CHECK(dim_v <= 512, "dim_v should be at most 512");
    TORCH_CHECK(head_q % head_k == 0, "number of heads in key/value must divide number of heads in query");

    DA_CHECK_SHAPE(q, total_q, head_q, dim);
    DA_CHECK_SHAPE(k, total_k, head_k, dim);
    DA_CHECK_SHAPE(cu_seq_k, batch + 1);
    TORCH_CHECK(q.stride(1) == dim && k.stride(1) == dim, "heads must be contiguous inside a token row");

    const at::cuda::CUDAGuard guard(q.device());
    auto stream = at::cuda::getCurrentCUDAStream().stream();

    da_decode_args_t a;
    std::memset(&a, 0, sizeof(a));
    a.struct_size = sizeof(a);
    a.is_bf16 = is_bf16;
    a.is_alibi = is_alibi;
    a.q = q.data_ptr();
    a.k = k.data_ptr();
    a.q_row_stride = q.stride(0);
    a.k_row_stride = k.stride(0);

    if (v_.has_value()) {
        const at::Tensor &v = v_.value();
        TORCH_CHECK(v.dtype() == k.dtype(), fp8_cache ? "key and value must have the same quantised dtype" : "query and value must have the same dtype");
        DA_CHECK_DEVICE(v);
        TORCH_CHECK(v.device() == q.device(), "all tensors must be on one device");
        TORCH_CHECK(v.stride(-1) == 1, "value must have contiguous last dimension");
        DA_CHECK_SHAPE(v, total_k, head_k, dim_v);
        TORCH_CHECK(v.stride(1) == dim_v, "heads must be contiguous inside a token row");
        a.v = v.data_ptr();
        a.v_row_stride = v.stride(0);
    }

    Outputs out;
    if (o_.has_value()) {
        out.o = o_.value();
        TORCH_CHECK(out.o.dtype() == q_dtype, "Output must have the same dtype as inputs");
        DA_CHECK_DEVICE(out.o);
        TORCH_CHECK(out.o.device() == q.device(), "all tensors must be on one device");
        TORCH_CHECK(out.o.stride(-1) == 1, "Output tensor must have contiguous last dimension");
        DA_CHECK_SHAPE(out.o, total_q, head_q, dim_v);
        TORCH_CHECK(out.o.stride(1) == dim_v, "heads must be contiguous inside a token row");
    } else {
        out.o = torch::empty({total_q, head_q, dim_v}, q.options());
    }
    a.o = out.o.data_ptr();
    a.o_row_stride = out.o.stride(0);
    if (want_lse) {
        out.lse = torch::empty({total_q, head_q}, q.options().dtype(torch::kFloat32));
        a.lse = out.lse.data_ptr<float>();
    }

    a.cu_seq_k = cu_seq_k.data_ptr<int32_t>();
    a.max_seq_k = max_seq_k;
    a.total_k = block_table ? 0u : (uint32_t)std::min<int64_t>(total_k, 0xFFFFFFFFll);  // a packed cache's rows are the batch's keys
    a.batch = batch;
    a.head_q = head_q;
    a.head_k = head_k;
    a.dim = dim;
    a.dim_v = dim_v;
    a.softmax_scale = softmax_scale.has_value() ? (float)softmax_scale.value() : 0.0f;
    a.stream = stream;
    if (fp8_cache) {
        TORCH_CHECK(v_.has_value(), "a quantised cache needs a value tensor");
        a.kv_dtype = int8_cache ? DA_KV_INT8 : DA_KV_FP8_E4M3;
        a.k_scale = (float)k_scale;
        a.v_scale = (float)v_scale;
    }
    if (block_table) {
        TORCH_CHECK(block_table->dtype() == torch::kInt32, "block_table must have dtype int32");
        TORCH_CHECK(block_table->is_cuda() && block_table->device() == q.device(), "all tensors must be on one device");
        TORCH_CHECK(block_table->dim() == 2 && block_table->size(0) == batch && block_table->stride(1) == 1,
                    "block_table must be [batch, blocks] with a contiguous last dimension");
        a.block_table = block_table->data_ptr<int32_t>();
        a.block_table_stride = block_table->stride(0);
        a.page_size = (int32_t)page_size;
    }

    // Split partials come from torch's caching allocator, which is ordered on the current stream: calls
    // on different streams of one device never share scratch, and nothing is allocated from the driver
    // once the allocator has warmed up (so the call can be captured in a CUDA graph).
    at::Tensor workspace;
    const size_t ws_bytes = da_decode_workspace_bytes(&a);
    if (ws_bytes > 0) {
        workspace = torch::empty({(int64_t)ws_bytes}, q.options().dtype(torch::kUInt8));
        a.workspace = workspace.data_ptr();
        a.workspace_bytes = ws_bytes;
    }
    const int rc = da_decode_fwd(&a);
    TORCH_CHECK(rc == DA_OK, "decoding_attn: ", da_status_string(rc), ": ", da_last_error());
    return out;
}

// Reference signature (decoding_torch.cpp:19-21).
at::Tensor fwd(const at::Tensor &q, const at::Tensor &k, std::optional<at::Tensor> v_, std::optional<at::Tensor> o_,
               const at::Tensor &cu_seq_k, const int64_t max_seq_k, const int64_t dim_v, const bool is_alibi) {
    return run(q, k, v_, o_, cu_seq_k, max_seq_k, dim_v, is_alibi, std::nullopt, false).o;
}

pybind11::object dmha_fwd(const at::Tensor &q, const at::Tensor &k, const at::Tensor &v, const at::Tensor &cu_seq_k,
                          int64_t max_seq_k, bool is_alibi, std::optional<double> softmax_scale,
                          std::optional<at::Tensor> out, bool return_lse, double k_scale, double v_scale) {
    TORCH_CHECK(v.dim() == 3, "value must be 3-D");
    Outputs r = run(q, k, v, out, cu_seq_k, max_seq_k, v.size(2), is_alibi, softmax_scale, return_lse, nullptr, 0,
                    k_scale, v_scale);
    if (return_lse) return pybind11::cast(std::make_tuple(r.o, r.lse));
    return pybind11::cast(r.o);
}

pybind11::object dmla_fwd(const at::Tensor &q, const at::Tensor &kv, const at::Tensor &cu_seq_k, int64_t max_seq_k,
                          int64_t dim_v, bool is_alibi, std::optional<double> softmax_scale,
                          std::optional<at::Tensor> out, bool return_lse) {
    // The reference's fwd() keeps is_alibi when v_ is None (csrc/torch/decoding_torch.cpp:19-21, :76-77).
    Outputs r = run(q, kv, std::nullopt, out, cu_seq_k, max_seq_k, dim_v, is_alibi, softmax_scale, return_lse);
    if (return_lse) return pybind11::cast(std::make_tuple(r.o, r.lse));
    return pybind11::cast(r.o);
}

// Paged cache: k_cache [num_pages, page_size, head_k, dim], v_cache the same with dim_v (or None for the
// latent-KV shape), block_table int32 [batch, blocks].  No counterpart in the reference's binding; its
// Python benchmark builds these layouts for the libraries it compares against
// (benchmarks/python/benchmark_decoding_attn.py:129-151, :182-190).
pybind11::object paged_fwd(const at::Tensor &q, const at::Tensor &k_cache, std::optional<at::Tensor> v_cache,
                           const at::Tensor &cu_seq_k, const at::Tensor &block_table, int64_t max_seq_k, int64_t dim_v,
                           bool is_alibi, std::optional<double> softmax_scale, std::optional<at::Tensor> out,
                           bool return_lse) {
    TORCH_CHECK(k_cache.dim() == 4 && k_cache.is_contiguous(), "k_cache must be a contiguous [pages, page_size, head_k, dim]");
    const int64_t page_size = k_cache.size(1);
    const at::Tensor k = k_cache.view({-1, k_cache.size(2), k_cache.size(3)});
    std::optional<at::Tensor> v;
    if (v_cache.has_value()) {
        TORCH_CHECK(v_cache->dim() == 4 && v_cache->is_contiguous() && v_cache->size(0) == k_cache.size(0) &&
                        v_cache->size(1) == page_size,
                    "v_cache must be a contiguous [pages, page_size, head_k, dim_v] like k_cache");
        v = v_cache->view({-1, v_cache->size(2), v_cache->size(3)});
    }
    Outputs r = run(q, k, v, out, cu_seq_k, max_seq_k, dim_v, is_alibi, softmax_scale, return_lse, &block_table, page_size);
    if (return_lse) return pybind11::cast(std::make_tuple(r.o, r.lse));
    return pybind11::cast(r.o);
}

// part_o fp32 [parts, rows..., dim_v], part_lse fp32 [parts, rows...] -> (o [rows..., dim_v], lse).
std::tuple<at::Tensor, at::Tensor> merge_partials(const at::Tensor &part_o, const at::Tensor &part_lse,
                                                  at::ScalarType out_dtype) {
    DA_CHECK_DEVICE(part_o);
    DA_CHECK_DEVICE(part_lse);
    DA_CHECK_CONTIGUOUS(part_o);
    DA_CHECK_CONTIGUOUS(part_lse);
    TORCH_CHECK(part_o.dtype() == torch::kFloat32 && part_lse.dtype() == torch::kFloat32, "partials must be fp32");
    TORCH_CHECK(out_dtype == torch::kFloat16 || out_dtype == torch::kBFloat16, "output must be fp16 or bf16");
    TORCH_CHECK(part_o.dim() >= 2 && part_lse.dim() == part_o.dim() - 1, "part_o [parts, ..., dim_v], part_lse [parts, ...]");
    const int64_t parts = part_o.size(0), dim_v = part_o.size(-1);
    const int64_t rows = part_lse.numel() / parts;
    TORCH_CHECK(part_o.numel() == parts * rows * dim_v, "part_o / part_lse shapes disagree");
    const at::cuda::CUDAGuard guard(part_o.device());
    auto out_shape = part_o.sizes().vec();
    out_shape.erase(out_shape.begin());
    at::Tensor o = torch::empty(out_shape, part_o.options().dtype(out_dtype));
    auto lse_shape = part_lse.sizes().vec();
    lse_shape.erase(lse_shape.begin());
    at::Tensor lse = torch::empty(lse_shape, part_lse.options());
    const int rc = da_merge_partials(part_o.data_ptr<float>(), part_lse.data_ptr<float>(), (int32_t)parts, rows,
                                     (int32_t)dim_v, rows * dim_v, dim_v, rows, 1, o.data_ptr(), nullptr,
                                     lse.data_ptr<float>(), out_dtype == torch::kBFloat16,
                                     at::cuda::getCurrentCUDAStream().stream());
    TORCH_CHECK(rc == DA_OK, "decoding_attn: ", da_status_string(rc), ": ", da_last_error());
    return {o, lse};
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    namespace py = pybind11;
    m.doc() = "Decoding-Attention (B200)";
    m.def("fwd", &fwd, "Forward pass", py::arg("q"), py::arg("k"), py::arg("v_"), py::arg("o_"), py::arg("cu_seq_k"),
          py::arg("max_seq_k"), py::arg("dim_v"), py::arg("is_alibi"));
    m.def("dmha_fwd", &dmha_fwd, "MHA/GQA/MQA decode", py::arg("q"), py::arg("k"), py::arg("v"), py::arg("cu_seq_k"),
          py::arg("max_seq_k"), py::arg("is_alibi") = false, py::arg("softmax_scale") = py::none(),
          py::arg("out") = py::none(), py::arg("return_lse") = false, py::arg("k_scale") = 1.0, py::arg("v_scale") = 1.0);
    m.def("dmla_fwd", &dmla_fwd, "MLA decode (latent KV)", py::arg("q"), py::arg("kv"), py::arg("cu_seq_k"),
          py::arg("max_seq_k"), py::arg("dim_v") = 512, py::arg("is_alibi") = false,
          py::arg("softmax_scale") = py::none(), py::arg("out") = py::none(), py::arg("return_lse") = false);
    m.def("paged_fwd", &paged_fwd, "Decode over a paged KV cache", py::arg("q"), py::arg("k_cache"), py::arg("v_cache"),
          py::arg("cu_seq_k"), py::arg("block_table"), py::arg("max_seq_k"), py::arg("dim_v"), py::arg("is_alibi") = false,
          py::arg("softmax_scale") = py::none(), py::arg("out") = py::none(), py::arg("return_lse") = false);
    m.def("merge_partials", &merge_partials, "LSE merge of key-range partials", py::arg("part_o"),
          py::arg("part_lse"), py::arg("out_dtype"));
    m.def("launch_count", []() { return da_launch_count(); });
    m.def("device_status", []() { return da_device_status(); });
}
