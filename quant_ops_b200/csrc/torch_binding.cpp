// Thin PyTorch binding: registers the reference's dispatcher ops (namespace quant_ops) and forwards tensors'
// pointers, sizes and the current CUDA stream to the C ABI.  No kernels and no arithmetic here.
//
// Schemas replaced (reference project paths):
//   quant_ops::flatquant_dynamic_quantize  src/quant_ops/ops/quantization/flatquant/kernels/cuda_quant_kernel.cu:407-413
//   quant_ops::int4_matmul                 src/quant_ops/ops/quantization/int4_matmul/kernels/cuda_int4_matmul_kernel.cu:207-214
// Only the CUDA dispatch key gets an implementation: CPU tensors raise, there is no fallback.
#include <ATen/ATen.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/library.h>

#include <tuple>

#include "quant_ops_b200.h"

namespace {

int to_qo_dtype(at::ScalarType t, const char* what) {
  switch (t) {
    case at::kFloat: return QO_F32;
    case at::kHalf: return QO_F16;
    case at::kBFloat16: return QO_BF16;
    default: TORCH_CHECK(false, what, " must be float32, float16 or bfloat16, got ", t);
  }
}

void check_status(int rc, const char* op) {
  TORCH_CHECK(rc == QO_OK, op, ": ", qo_status_string(rc), ": ", qo_last_error());
}

void* current_stream() { return static_cast<void*>(c10::cuda::getCurrentCUDAStream().stream()); }

// rows of a 2-D tensor must be unit-stride; anything else is copied once
at::Tensor row_major(const at::Tensor& t) {
  if (t.dim() == 2 && t.stride(1) == 1 && (t.size(0) <= 1 || t.stride(0) >= t.size(1))) return t;
  return t.contiguous();
}

// scale_dtype: dtype of the returned per-token scales; float32 (what the reference's CUDA op returns) when absent
std::tuple<at::Tensor, at::Tensor> flatquant_dynamic_quantize_ex(const at::Tensor& input, const at::Tensor& left_trans,
                                                                 const at::Tensor& right_trans, double clip_ratio,
                                                                 bool pack_int32,
                                                                 c10::optional<at::ScalarType> scale_dtype_opt) {
  const at::ScalarType scale_dtype = scale_dtype_opt.has_value() ? *scale_dtype_opt : at::kFloat;
  const int sdt = to_qo_dtype(scale_dtype, "scale_dtype");
  TORCH_CHECK(input.is_cuda() && left_trans.is_cuda() && right_trans.is_cuda(),
              "flatquant_dynamic_quantize: all tensors must be CUDA tensors");
  TORCH_CHECK(left_trans.dim() == 2 && left_trans.size(0) == left_trans.size(1), "left_trans must be square [M, M]");
  TORCH_CHECK(right_trans.dim() == 2 && right_trans.size(0) == right_trans.size(1), "right_trans must be square [N, N]");
  TORCH_CHECK(left_trans.scalar_type() == input.scalar_type() && right_trans.scalar_type() == input.scalar_type(),
              "left_trans and right_trans must have the dtype of the input (", input.scalar_type(), ")");
  TORCH_CHECK(left_trans.device() == input.device() && right_trans.device() == input.device(),
              "all tensors must be on the same device");
  const int64_t m = left_trans.size(0), n = right_trans.size(0), features = m * n;
  TORCH_CHECK(input.dim() == 2 || input.dim() == 3, "input must be [tokens, M*N] or [tokens, M, N]");
  at::Tensor x2 = input.dim() == 3 ? input.reshape({input.size(0), -1}) : input;
  TORCH_CHECK(x2.size(-1) == features, "Input last dimension must equal M*N");
  TORCH_CHECK(features % 8 == 0 || !pack_int32, "Features must be divisible by 8 for int32 packing");
  const int dt = to_qo_dtype(input.scalar_type(), "input");
  c10::cuda::CUDAGuard guard(input.device());
  x2 = row_major(x2);
  at::Tensor left = left_trans.contiguous(), right = right_trans.contiguous();
  const int64_t tokens = x2.size(0);
  at::Tensor codes = pack_int32 ? at::empty({tokens, features / 8}, input.options().dtype(at::kInt))
                                : at::empty({tokens, features}, input.options().dtype(at::kChar));
  at::Tensor scales = at::empty({tokens}, input.options().dtype(scale_dtype));
  check_status(qo_flatquant_quantize(x2.data_ptr(), tokens > 1 ? x2.stride(0) : features, left.data_ptr(),
                                     right.data_ptr(), codes.data_ptr(), scales.data_ptr(), tokens, (int)m, (int)n,
                                     (float)clip_ratio, dt, pack_int32 ? 1 : 0, sdt, current_stream()),
               "flatquant_dynamic_quantize");
  return {codes, scales};
}

std::tuple<at::Tensor, at::Tensor> flatquant_dynamic_quantize(const at::Tensor& input, const at::Tensor& left_trans,
                                                              const at::Tensor& right_trans, double clip_ratio,
                                                              bool pack_int32) {
  return flatquant_dynamic_quantize_ex(input, left_trans, right_trans, clip_ratio, pack_int32, c10::nullopt);
}

std::tuple<at::Tensor, at::Tensor> int4_matmul_ex(const at::Tensor& a, const at::Tensor& b, const at::Tensor& scale_a,
                                                  const at::Tensor& scale_b, at::ScalarType out_dtype,
                                                  bool return_acc) {
  TORCH_CHECK(a.is_cuda(), "a_packed must be on CUDA");
  TORCH_CHECK(b.is_cuda(), "b_packed must be on CUDA");
  TORCH_CHECK(scale_a.is_cuda(), "scale_a must be on CUDA");
  TORCH_CHECK(scale_b.is_cuda(), "scale_b must be on CUDA");
  TORCH_CHECK(a.scalar_type() == at::kInt, "a_packed must be int32");
  TORCH_CHECK(b.scalar_type() == at::kInt, "b_packed must be int32");
  TORCH_CHECK(scale_a.scalar_type() == at::kFloat, "scale_a must be float32");
  TORCH_CHECK(scale_b.scalar_type() == at::kFloat, "scale_b must be float32");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2, "a_packed and b_packed must be 2-D");
  TORCH_CHECK(out_dtype == at::kHalf || out_dtype == at::kBFloat16, "out_dtype must be float16 or bfloat16");
  const int64_t t = a.size(0), kp = a.size(1), n = b.size(1);
  TORCH_CHECK(b.size(0) == kp, "Matrix dimensions mismatch");
  TORCH_CHECK(scale_a.numel() == t, "scale_a dimension mismatch");
  TORCH_CHECK(scale_b.numel() == n, "scale_b dimension mismatch");
  c10::cuda::CUDAGuard guard(a.device());
  at::Tensor a2 = row_major(a);
  // b may be the canonical [K/8, N] layout or the transposed view of a [N, K/8] weight; both go through as strides
  at::Tensor b2 = (b.stride(0) == 1 || b.stride(1) == 1 || b.numel() == 0) ? b : b.contiguous();
  at::Tensor sa = scale_a.reshape({-1}).contiguous(), sb = scale_b.reshape({-1}).contiguous();
  at::Tensor out = at::empty({t, n}, a.options().dtype(out_dtype));
  at::Tensor acc = return_acc ? at::empty({t, n}, a.options().dtype(at::kInt)) : at::Tensor();
  const size_t ws_bytes = qo_int4_matmul_workspace_bytes(t, kp * 8, n);
  at::Tensor ws = at::empty({(int64_t)ws_bytes}, a.options().dtype(at::kByte));
  check_status(qo_int4_matmul(a2.data_ptr<int32_t>(), t > 1 ? a2.stride(0) : kp, b2.data_ptr<int32_t>(), b2.stride(0),
                              b2.stride(1), sa.data_ptr<float>(), sb.data_ptr<float>(), out.data_ptr(),
                              out_dtype == at::kHalf ? QO_F16 : QO_BF16, t, kp * 8, n,
                              return_acc ? acc.data_ptr<int32_t>() : nullptr, ws_bytes ? ws.data_ptr() : nullptr, ws_bytes,
                              current_stream()),
               "int4_matmul");
  if (!return_acc) acc = at::empty({0}, a.options().dtype(at::kInt));
  return {out, acc};
}

at::Tensor int4_matmul(const at::Tensor& a, const at::Tensor& b, const at::Tensor& scale_a, const at::Tensor& scale_b) {
  return std::get<0>(int4_matmul_ex(a, b, scale_a, scale_b, at::kHalf, false));
}

at::Tensor dequantize_int4(const at::Tensor& quantized, const at::Tensor& scales, bool packed_int32) {
  TORCH_CHECK(quantized.is_cuda() && scales.is_cuda(), "dequantize_int4: tensors must be CUDA tensors");
  TORCH_CHECK(quantized.dim() == 2, "dequantize_int4: quantized must be 2-D");
  TORCH_CHECK(quantized.scalar_type() == (packed_int32 ? at::kInt : at::kChar),
              "dequantize_int4: quantized must be ", packed_int32 ? "int32 (packed)" : "int8");
  const int64_t tokens = quantized.size(0), features = quantized.size(1) * (packed_int32 ? 8 : 1);
  TORCH_CHECK(scales.numel() == tokens, "dequantize_int4: one scale per token expected");
  const int sdt = to_qo_dtype(scales.scalar_type(), "scales");
  c10::cuda::CUDAGuard guard(quantized.device());
  at::Tensor q = quantized.contiguous(), s = scales.reshape({-1}).contiguous();
  at::Tensor out = at::empty({tokens, features}, quantized.options().dtype(at::kFloat));
  check_status(qo_dequantize_int4(q.data_ptr(), s.data_ptr(), out.data_ptr<float>(), tokens, features,
                                  packed_int32 ? 1 : 0, sdt, current_stream()),
               "dequantize_int4");
  return out;
}

at::Tensor w4a4_linear(const at::Tensor& x, const at::Tensor& left_trans, const at::Tensor& right_trans,
                       const at::Tensor& w_packed, const at::Tensor& w_scale, const c10::optional<at::Tensor>& bias,
                       double clip_ratio, c10::optional<at::ScalarType> out_dtype_opt) {
  TORCH_CHECK(x.is_cuda() && left_trans.is_cuda() && right_trans.is_cuda() && w_packed.is_cuda() && w_scale.is_cuda(),
              "w4a4_linear: all tensors must be CUDA tensors");
  TORCH_CHECK(x.dim() == 2, "w4a4_linear: x must be [tokens, K]");
  const int64_t m = left_trans.size(0), n = right_trans.size(0), k = m * n;
  TORCH_CHECK(x.size(1) == k, "w4a4_linear: x last dimension must equal M*N");
  TORCH_CHECK(left_trans.scalar_type() == x.scalar_type() && right_trans.scalar_type() == x.scalar_type(),
              "w4a4_linear: transforms must have the dtype of x");
  TORCH_CHECK(w_packed.dim() == 2 && w_packed.scalar_type() == at::kInt && w_packed.size(1) * 8 == k,
              "w4a4_linear: w_packed must be int32 [n_out, K/8]");
  TORCH_CHECK(w_scale.scalar_type() == at::kFloat && w_scale.numel() == w_packed.size(0),
              "w4a4_linear: w_scale must be float32 [n_out]");
  const at::ScalarType out_dtype = out_dtype_opt.has_value() ? *out_dtype_opt : (x.scalar_type() == at::kBFloat16 ? at::kBFloat16 : at::kHalf);
  TORCH_CHECK(out_dtype == at::kHalf || out_dtype == at::kBFloat16, "w4a4_linear: out_dtype must be float16 or bfloat16");
  const int dt = to_qo_dtype(x.scalar_type(), "x");
  c10::cuda::CUDAGuard guard(x.device());
  at::Tensor x2 = row_major(x), left = left_trans.contiguous(), right = right_trans.contiguous();
  at::Tensor w = w_packed.contiguous(), ws_ = w_scale.reshape({-1}).contiguous();
  at::Tensor b;
  if (bias.has_value() && bias->defined()) {
    TORCH_CHECK(bias->numel() == w.size(0), "w4a4_linear: bias must have n_out elements");
    b = bias->to(out_dtype).contiguous();
  }
  const int64_t tokens = x2.size(0), n_out = w.size(0);
  at::Tensor out = at::empty({tokens, n_out}, x.options().dtype(out_dtype));
  const size_t ws_bytes = qo_w4a4_linear_workspace_bytes(tokens, k, n_out);
  at::Tensor ws = at::empty({(int64_t)ws_bytes}, x.options().dtype(at::kByte));
  check_status(qo_w4a4_linear(x2.data_ptr(), tokens > 1 ? x2.stride(0) : k, left.data_ptr(), right.data_ptr(),
                              w.data_ptr<int32_t>(), ws_.data_ptr<float>(), b.defined() ? b.data_ptr() : nullptr,
                              out.data_ptr(), tokens, (int)m, (int)n, n_out, (float)clip_ratio, dt,
                              out_dtype == at::kHalf ? QO_F16 : QO_BF16, ws_bytes ? ws.data_ptr() : nullptr, ws_bytes,
                              current_stream()),
               "w4a4_linear");
  return out;
}

at::Tensor prepare_weights(const at::Tensor& w_packed) {
  TORCH_CHECK(w_packed.is_cuda() && w_packed.dim() == 2 && w_packed.scalar_type() == at::kInt,
              "prepare_weights: int32 CUDA [n_out, K/8] expected");
  c10::cuda::CUDAGuard guard(w_packed.device());
  at::Tensor w = w_packed.contiguous();
  const int64_t n_out = w.size(0), k = w.size(1) * 8;
  at::Tensor out = at::empty({(int64_t)qo_prepared_weights_bytes(n_out, k)}, w.options().dtype(at::kByte));
  check_status(qo_prepare_weights(w.data_ptr<int32_t>(), out.data_ptr(), n_out, k, current_stream()), "prepare_weights");
  return out;
}

at::Tensor w4a4_linear_prepared(const at::Tensor& x, const at::Tensor& left_trans, const at::Tensor& right_trans,
                                const at::Tensor& w_packed, const at::Tensor& w_prepared, const at::Tensor& w_scale,
                                const c10::optional<at::Tensor>& bias, double clip_ratio,
                                c10::optional<at::ScalarType> out_dtype_opt) {
  TORCH_CHECK(x.is_cuda() && left_trans.is_cuda() && right_trans.is_cuda() && w_packed.is_cuda() && w_prepared.is_cuda() &&
                  w_scale.is_cuda(), "w4a4_linear_prepared: all tensors must be CUDA tensors");
  TORCH_CHECK(x.dim() == 2, "w4a4_linear_prepared: x must be [tokens, K]");
  const int64_t m = left_trans.size(0), n = right_trans.size(0), k = m * n;
  TORCH_CHECK(x.size(1) == k, "w4a4_linear_prepared: x last dimension must equal M*N");
  TORCH_CHECK(left_trans.scalar_type() == x.scalar_type() && right_trans.scalar_type() == x.scalar_type(),
              "w4a4_linear_prepared: transforms must have the dtype of x");
  TORCH_CHECK(w_packed.dim() == 2 && w_packed.scalar_type() == at::kInt && w_packed.size(1) * 8 == k,
              "w4a4_linear_prepared: w_packed must be int32 [n_out, K/8]");
  TORCH_CHECK(w_prepared.dim() == 1 && w_prepared.scalar_type() == at::kByte && w_prepared.is_contiguous() &&
                  w_prepared.numel() == (int64_t)qo_prepared_weights_bytes(w_packed.size(0), k),
              "w4a4_linear_prepared: w_prepared must be the byte tensor made by prepare_weights for these weights");
  TORCH_CHECK(w_scale.scalar_type() == at::kFloat && w_scale.numel() == w_packed.size(0),
              "w4a4_linear_prepared: w_scale must be float32 [n_out]");
  const at::ScalarType out_dtype = out_dtype_opt.has_value() ? *out_dtype_opt : (x.scalar_type() == at::kBFloat16 ? at::kBFloat16 : at::kHalf);
  TORCH_CHECK(out_dtype == at::kHalf || out_dtype == at::kBFloat16, "w4a4_linear_prepared: out_dtype must be float16 or bfloat16");
  const int dt = to_qo_dtype(x.scalar_type(), "x");
  c10::cuda::CUDAGuard guard(x.device());
  at::Tensor x2 = row_major(x), left = left_trans.contiguous(), right = right_trans.contiguous();
  at::Tensor w = w_packed.contiguous(), ws_ = w_scale.reshape({-1}).contiguous();
  at::Tensor b;
  if (bias.has_value() && bias->defined()) {
    TORCH_CHECK(bias->numel() == w.size(0), "w4a4_linear_prepared: bias must have n_out elements");
    b = bias->to(out_dtype).contiguous();
  }
  const int64_t tokens = x2.size(0), n_out = w.size(0);
  at::Tensor out = at::empty({tokens, n_out}, x.options().dtype(out_dtype));
  const size_t ws_bytes = qo_w4a4_linear_prepared_workspace_bytes(tokens, k, n_out);
  at::Tensor ws = at::empty({(int64_t)ws_bytes}, x.options().dtype(at::kByte));
  check_status(qo_w4a4_linear_prepared(x2.data_ptr(), tokens > 1 ? x2.stride(0) : k, left.data_ptr(), right.data_ptr(),
                                       w.data_ptr<int32_t>(), w_prepared.data_ptr(), ws_.data_ptr<float>(),
                                       b.defined() ? b.data_ptr() : nullptr, out.data_ptr(), tokens, (int)m, (int)n, n_out,
                                       (float)clip_ratio, dt, out_dtype == at::kHalf ? QO_F16 : QO_BF16,
                                       ws_bytes ? ws.data_ptr() : nullptr, ws_bytes, current_stream()),
               "w4a4_linear_prepared");
  return out;
}

at::Tensor pack_int4(const at::Tensor& codes) {
  TORCH_CHECK(codes.is_cuda() && codes.scalar_type() == at::kChar && codes.dim() == 2, "pack_int4: int8 CUDA [rows, features] expected");
  TORCH_CHECK(codes.size(1) % 8 == 0, "features (", codes.size(1), ") must be divisible by 8");
  c10::cuda::CUDAGuard guard(codes.device());
  at::Tensor c = codes.contiguous();
  at::Tensor out = at::empty({c.size(0), c.size(1) / 8}, codes.options().dtype(at::kInt));
  check_status(qo_pack_int4(c.data_ptr<int8_t>(), out.data_ptr<int32_t>(), c.size(0), c.size(1), current_stream()), "pack_int4");
  return out;
}

at::Tensor unpack_int4(const at::Tensor& packed) {
  TORCH_CHECK(packed.is_cuda() && packed.scalar_type() == at::kInt && packed.dim() == 2, "unpack_int4: int32 CUDA [rows, features/8] expected");
  c10::cuda::CUDAGuard guard(packed.device());
  at::Tensor p = packed.contiguous();
  at::Tensor out = at::empty({p.size(0), p.size(1) * 8}, packed.options().dtype(at::kChar));
  check_status(qo_unpack_int4(p.data_ptr<int32_t>(), out.data_ptr<int8_t>(), p.size(0), p.size(1) * 8, current_stream()), "unpack_int4");
  return out;
}

std::tuple<at::Tensor, at::Tensor> quantize_weights_int4(const at::Tensor& w) {
  TORCH_CHECK(w.is_cuda() && w.dim() == 2, "quantize_weights_int4: CUDA [rows, k] expected");
  TORCH_CHECK(w.size(1) % 8 == 0, "k (", w.size(1), ") must be divisible by 8");
  c10::cuda::CUDAGuard guard(w.device());
  at::Tensor wf = w.to(at::kFloat).contiguous();
  at::Tensor packed = at::empty({wf.size(0), wf.size(1) / 8}, w.options().dtype(at::kInt));
  at::Tensor scale = at::empty({wf.size(0)}, w.options().dtype(at::kFloat));
  check_status(qo_quantize_weights_int4(wf.data_ptr<float>(), packed.data_ptr<int32_t>(), scale.data_ptr<float>(),
                                        wf.size(0), wf.size(1), current_stream()),
               "quantize_weights_int4");
  return {packed, scale};
}

}  // namespace

TORCH_LIBRARY(quant_ops, m) {
  m.def("flatquant_dynamic_quantize(Tensor input, Tensor left_trans, Tensor right_trans, float clip_ratio=1, bool pack_int32=False) -> (Tensor, Tensor)");
  m.def("flatquant_dynamic_quantize_ex(Tensor input, Tensor left_trans, Tensor right_trans, float clip_ratio=1, bool pack_int32=False, ScalarType? scale_dtype=None) -> (Tensor, Tensor)");
  m.def("int4_matmul(Tensor a, Tensor b, Tensor scale_a, Tensor scale_b) -> Tensor");
  m.def("int4_matmul_ex(Tensor a, Tensor b, Tensor scale_a, Tensor scale_b, ScalarType out_dtype, bool return_acc=False) -> (Tensor, Tensor)");
  m.def("dequantize_int4(Tensor quantized, Tensor scales, bool packed_int32=False) -> Tensor");
  m.def("w4a4_linear(Tensor x, Tensor left_trans, Tensor right_trans, Tensor w_packed, Tensor w_scale, Tensor? bias=None, float clip_ratio=1, ScalarType? out_dtype=None) -> Tensor");
  m.def("prepare_weights(Tensor w_packed) -> Tensor");
  m.def("w4a4_linear_prepared(Tensor x, Tensor left_trans, Tensor right_trans, Tensor w_packed, Tensor w_prepared, Tensor w_scale, Tensor? bias=None, float clip_ratio=1, ScalarType? out_dtype=None) -> Tensor");
  m.def("pack_int4(Tensor codes) -> Tensor");
  m.def("unpack_int4(Tensor packed) -> Tensor");
  m.def("quantize_weights_int4(Tensor w) -> (Tensor, Tensor)");
}

TORCH_LIBRARY_IMPL(quant_ops, CUDA, m) {
  m.impl("flatquant_dynamic_quantize", &flatquant_dynamic_quantize);
  m.impl("flatquant_dynamic_quantize_ex", &flatquant_dynamic_quantize_ex);
  m.impl("int4_matmul", &int4_matmul);
  m.impl("int4_matmul_ex", &int4_matmul_ex);
  m.impl("dequantize_int4", &dequantize_int4);
  m.impl("w4a4_linear", &w4a4_linear);
  m.impl("prepare_weights", &prepare_weights);
  m.impl("w4a4_linear_prepared", &w4a4_linear_prepared);
  m.impl("pack_int4", &pack_int4);
  m.impl("unpack_int4", &unpack_int4);
  m.impl("quantize_weights_int4", &quantize_weights_int4);
}
