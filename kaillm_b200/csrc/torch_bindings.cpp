// `_C_gguf` PyTorch extension: the same op schemas the reference registers
// (vllm_gguf_plugin/csrc/torch_bindings.cpp:22-61), implemented by calling the libkq C ABI
// (include/kq_gguf.h).  torch supplies device memory, the current stream and the dispatcher; all
// arithmetic happens behind the C ABI.
//
// Differences from the reference bindings, on purpose:
//   - outputs come from at::empty (the kernels write every element; the reference memsets with new_zeros);
//   - an unsupported GGML type raises instead of silently returning zeros
//     (reference: switch without default, csrc/gguf/gguf_kernel.cu:119-215);
//   - the MoE ops are declared, so the unmodified Python wrapper can register its fake implementations
//     (vllm_gguf_plugin/ops.py:110-175), but raise: they are outside this library's scope.
#include <Python.h>

#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include "../../include/kq_gguf.h"

namespace {

int kq_dtype_of(at::ScalarType t, const char* what) {
  switch (t) {
    case at::kFloat: return KQ_F32;
    case at::kHalf: return KQ_F16;
    case at::kBFloat16: return KQ_BF16;
    default: TORCH_CHECK(false, what, ": dtype must be float32, float16 or bfloat16, got ", t);
  }
}

void check_weight(const at::Tensor& W, const char* fn) {
  TORCH_CHECK(W.is_cuda(), fn, ": W must be a CUDA tensor");
  TORCH_CHECK(W.scalar_type() == at::kByte, fn, ": W must be uint8 GGUF wire bytes");
  TORCH_CHECK(W.is_contiguous(), fn, ": W must be contiguous");
}

at::Tensor mul_mat_impl(bool mmq, const at::Tensor& W, const at::Tensor& X, int64_t type, int64_t row) {
  const char* fn = mmq ? "ggml_mul_mat_a8" : "ggml_mul_mat_vec_a8";
  check_weight(W, fn);
  TORCH_CHECK(X.is_cuda() && X.dim() == 2, fn, ": X must be a 2-D CUDA tensor");
  TORCH_CHECK(X.get_device() == W.get_device(), fn, ": W and X are on different devices");
  TORCH_CHECK(X.stride(1) == 1, fn, ": X must be contiguous along its last dimension");
  const int64_t m = X.size(0), k = X.size(1);
  const int xdt = kq_dtype_of(X.scalar_type(), fn);
  int blk = 0, bytes = 0;
  TORCH_CHECK(kq_block_geometry((int)type, &blk, &bytes) == KQ_OK, fn, ": ", kq_last_error());
  TORCH_CHECK(k % blk == 0, fn, ": X.size(1)=", k, " is not a multiple of the block size ", blk);
  TORCH_CHECK(row >= 0 && W.numel() >= row * (k / blk) * bytes, fn, ": W holds fewer than `row` rows of K=", k);
  const c10::cuda::CUDAGuard guard(X.device());
  at::Tensor Y = at::empty({m, row}, X.options());
  if (m == 0 || row == 0) return Y;
  const size_t ws = kq_workspace_bytes((int)type, m, row, k);
  at::Tensor scratch = at::empty({(int64_t)ws}, W.options());
  auto stream = at::cuda::getCurrentCUDAStream(X.get_device()).stream();
  auto fnp = mmq ? kq_mul_mat_a8 : kq_mul_mat_vec_a8;
  const int rc = fnp(W.data_ptr(), (int)type, row, k, X.data_ptr(), xdt, m, X.stride(0), Y.data_ptr(), xdt,
                     Y.stride(0), scratch.data_ptr(), ws, (void*)stream);
  TORCH_CHECK(rc == KQ_OK, fn, ": ", kq_last_error());
  return Y;
}

at::Tensor ggml_mul_mat_vec_a8(const at::Tensor& W, const at::Tensor& X, int64_t type, c10::SymInt row) {
  return mul_mat_impl(false, W, X, type, row.expect_int());
}

at::Tensor ggml_mul_mat_a8(const at::Tensor& W, const at::Tensor& X, int64_t type, c10::SymInt row) {
  return mul_mat_impl(true, W, X, type, row.expect_int());
}

at::Tensor ggml_dequantize(const at::Tensor& W, int64_t type, c10::SymInt m_, c10::SymInt n_,
                           std::optional<at::ScalarType> dtype) {
  const char* fn = "ggml_dequantize";
  check_weight(W, fn);
  const int64_t m = m_.expect_int(), n = n_.expect_int();
  const at::ScalarType dt = dtype.value_or(at::kHalf);
  const int odt = kq_dtype_of(dt, fn);
  int blk = 0, bytes = 0;
  TORCH_CHECK(kq_block_geometry((int)type, &blk, &bytes) == KQ_OK, fn, ": ", kq_last_error());
  TORCH_CHECK(m >= 0 && n >= 0 && (m * n) % blk == 0, fn, ": m*n must be a multiple of the block size ", blk);
  TORCH_CHECK(W.numel() >= (m * n) / blk * bytes, fn, ": W holds fewer than m*n weights");
  const c10::cuda::CUDAGuard guard(W.device());
  at::Tensor DW = at::empty({m, n}, W.options().dtype(dt));
  if (m * n == 0) return DW;
  auto stream = at::cuda::getCurrentCUDAStream(W.get_device()).stream();
  const int rc = kq_dequantize(W.data_ptr(), (int)type, m * n, DW.data_ptr(), odt, (void*)stream);
  TORCH_CHECK(rc == KQ_OK, fn, ": ", kq_last_error());
  return DW;
}

// W: [E, row, row bytes] (or any contiguous uint8 tensor holding E matrices back to back)
at::Tensor moe_impl(bool block, const at::Tensor& X, const at::Tensor& W, const at::Tensor& ids, const at::Tensor* expert_ids,
                    const at::Tensor* num_post_padded, int64_t type, int64_t row, int64_t top_k, int64_t tokens) {
  const char* fn = block ? "ggml_moe_a8" : "ggml_moe_a8_vec";
  check_weight(W, fn);
  TORCH_CHECK(X.is_cuda() && X.dim() == 2, fn, ": X must be a 2-D CUDA tensor");
  TORCH_CHECK(X.get_device() == W.get_device(), fn, ": W and X are on different devices");
  TORCH_CHECK(X.stride(1) == 1, fn, ": X must be contiguous along its last dimension");
  TORCH_CHECK(tokens >= 0 && tokens <= X.size(0), fn, ": `tokens` exceeds X.size(0)");
  TORCH_CHECK(top_k > 0 && row >= 0, fn, ": top_k must be positive");
  const int64_t k = X.size(1);
  const int xdt = kq_dtype_of(X.scalar_type(), fn);
  int blk = 0, bytes = 0;
  TORCH_CHECK(kq_block_geometry((int)type, &blk, &bytes) == KQ_OK, fn, ": ", kq_last_error());
  TORCH_CHECK(k % blk == 0, fn, ": X.size(1)=", k, " is not a multiple of the block size ", blk);
  const int64_t per_expert = row * (k / blk) * bytes;
  TORCH_CHECK(per_expert > 0 && W.numel() % per_expert == 0, fn, ": W is not a whole number of [row, K] matrices");
  const int64_t experts = W.numel() / per_expert;
  auto as_i32 = [&](const at::Tensor& t, const char* name) {
    TORCH_CHECK(t.is_cuda() && t.get_device() == X.get_device(), fn, ": ", name, " must be on X's device");
    return t.scalar_type() == at::kInt && t.is_contiguous() ? t : t.to(at::kInt).contiguous();
  };
  const c10::cuda::CUDAGuard guard(X.device());
  at::Tensor Y = at::zeros({tokens * top_k, row}, X.options());   // rows nobody writes read as zero, as in the reference
  if (tokens == 0 || row == 0) return Y;
  const at::Tensor ids32 = as_i32(ids, block ? "sorted_token_ids" : "topk_ids");
  const size_t ws = kq_workspace_bytes((int)type, tokens, row, k);
  at::Tensor scratch = at::empty({(int64_t)ws}, W.options());
  auto stream = at::cuda::getCurrentCUDAStream(X.get_device()).stream();
  int rc;
  if (block) {
    const at::Tensor e32 = as_i32(*expert_ids, "expert_ids"), n32 = as_i32(*num_post_padded, "num_tokens_post_padded");
    TORCH_CHECK(n32.numel() >= 1, fn, ": num_tokens_post_padded is empty");
    TORCH_CHECK(e32.numel() * kq_moe_block_size((int)type) >= ids32.numel(), fn, ": expert_ids has fewer entries than blocks of sorted tokens");
    rc = kq_moe_a8(W.data_ptr(), (int)type, experts, row, k, X.data_ptr(), xdt, tokens, X.stride(0), ids32.data_ptr<int32_t>(),
                   ids32.numel(), e32.data_ptr<int32_t>(), n32.data_ptr<int32_t>(), (int)top_k, Y.data_ptr(), xdt, Y.stride(0),
                   scratch.data_ptr(), ws, (void*)stream);
  } else {
    TORCH_CHECK(ids32.numel() >= tokens * top_k, fn, ": topk_ids has fewer than tokens * top_k entries");
    rc = kq_moe_a8_vec(W.data_ptr(), (int)type, experts, row, k, X.data_ptr(), xdt, tokens, X.stride(0), ids32.data_ptr<int32_t>(),
                       (int)top_k, Y.data_ptr(), xdt, Y.stride(0), scratch.data_ptr(), ws, (void*)stream);
  }
  TORCH_CHECK(rc == KQ_OK, fn, ": ", kq_last_error());
  return Y;
}

at::Tensor ggml_moe_a8(const at::Tensor& X, const at::Tensor& W, const at::Tensor& sorted_token_ids, const at::Tensor& expert_ids,
                       const at::Tensor& num_tokens_post_padded, int64_t type, c10::SymInt row, c10::SymInt top_k,
                       c10::SymInt tokens) {
  return moe_impl(true, X, W, sorted_token_ids, &expert_ids, &num_tokens_post_padded, type, row.expect_int(), top_k.expect_int(),
                  tokens.expect_int());
}

at::Tensor ggml_moe_a8_vec(const at::Tensor& X, const at::Tensor& W, const at::Tensor& topk_ids, int64_t top_k, int64_t type,
                           c10::SymInt row, c10::SymInt tokens) {
  return moe_impl(false, X, W, topk_ids, nullptr, nullptr, type, row.expect_int(), top_k, tokens.expect_int());
}

int64_t ggml_moe_get_block_size(int64_t type) { return kq_moe_block_size((int)type); }

}  // namespace

TORCH_LIBRARY(_C_gguf, ops) {
  ops.def("ggml_dequantize(Tensor W, int type, SymInt m, SymInt n, ScalarType? dtype) -> Tensor");
  ops.def("ggml_mul_mat_vec_a8(Tensor W, Tensor X, int type, SymInt row) -> Tensor");
  ops.def("ggml_mul_mat_a8(Tensor W, Tensor X, int type, SymInt row) -> Tensor");
  ops.def(
      "ggml_moe_a8(Tensor X, Tensor W, Tensor sorted_token_ids, Tensor expert_ids, Tensor "
      "num_tokens_post_padded, int type, SymInt row, SymInt top_k, SymInt tokens) -> Tensor");
  ops.def("ggml_moe_a8_vec(Tensor X, Tensor W, Tensor topk_ids, int top_k, int type, SymInt row, SymInt tokens) -> Tensor");
  ops.def("ggml_moe_get_block_size(int type) -> int");
}

TORCH_LIBRARY_IMPL(_C_gguf, CUDA, ops) {
  ops.impl("ggml_dequantize", &ggml_dequantize);
  ops.impl("ggml_mul_mat_vec_a8", &ggml_mul_mat_vec_a8);
  ops.impl("ggml_mul_mat_a8", &ggml_mul_mat_a8);
  ops.impl("ggml_moe_a8", &ggml_moe_a8);
  ops.impl("ggml_moe_a8_vec", &ggml_moe_a8_vec);
}

TORCH_LIBRARY_IMPL(_C_gguf, CompositeExplicitAutograd, ops) {
  ops.impl("ggml_moe_get_block_size", &ggml_moe_get_block_size);
}

static struct PyModuleDef kq_module_def = {PyModuleDef_HEAD_INIT, "_C_gguf", nullptr, -1, nullptr};

extern "C" PyObject* PyInit__C_gguf(void) { return PyModule_Create(&kq_module_def); }
