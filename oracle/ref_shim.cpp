// C-ABI shim over the reference's OWN CPU operators, compiled from the reference sources
// where they lie (nothing is copied): the include path points into the anyGPU checkout.
//
// TEST INFRASTRUCTURE ONLY: used to validate the restated oracle and as the timed CPU
// baseline. The shipped library never loads it.
//
// Wrapped reference functions:
//   tensor_linear<float32,CPU>               srcs/ops/mm_ops.hpp:206-232 (-> tensor_mm :11-45)
//   tensor_causal_conv1d<float32>(CPU)       srcs/fused/causal_conv1d.hpp:24-87
//   tensor_zamba_gated_rmsnorm<float32,CPU>  srcs/models/zamba2/zamba_gated_rmsnorm.hpp:9-23
//   tensor_silu / tensor_rms_norm            srcs/ops/math_ops.hpp:16-35, srcs/ops/norm_ops.hpp:134-194

#include "tensor.hpp"
#include "core_concepts.hpp"
#include "ops.hpp"
#include "causal_conv1d.hpp"
#include "zamba_gated_rmsnorm.hpp"

#include <cstring>

namespace {
Tensor<float32, CPU> make(const float* src, const std::vector<int64>& shape)
{
	Tensor<float32, CPU> t(shape);
	std::memcpy(t.buffer(), src, sizeof(float) * t.numel());
	return t;
}
}

extern "C" {

void ref_linear_f32(const float* x, const float* w, float* y, long long M, long long K, long long N)
{
	auto xt = make(x, { M, K });
	auto wt = make(w, { K, N });
	auto yt = tensor_linear(xt, wt);
	std::memcpy(y, yt.buffer(), sizeof(float) * M * N);
}

void ref_causal_conv1d_f32(const float* x, const float* w, const float* b, float* y,
	long long B, long long D, long long S, long long W)
{
	auto xt = make(x, { B, D, S });
	auto wt = make(w, { D, W });
	auto bt = make(b, { D });
	auto yt = tensor_causal_conv1d(xt, wt, bt);
	std::memcpy(y, yt.buffer(), sizeof(float) * B * D * S);
}

void ref_gated_rmsnorm_f32(const float* x, const float* z, const float* w, float* y,
	long long rows, long long d, int gsize, float eps)
{
	auto xt = make(x, { rows, d });
	auto zt = make(z, { rows, d });
	auto wt = make(w, { d });
	auto yt = tensor_zamba_gated_rmsnorm<float32, CPU>(xt, zt, wt, gsize, eps);
	std::memcpy(y, yt.buffer(), sizeof(float) * rows * d);
}

void ref_silu_f32(const float* x, float* y, long long n)
{
	auto xt = make(x, { n });
	auto yt = tensor_silu(xt);
	std::memcpy(y, yt.buffer(), sizeof(float) * n);
}

void ref_rms_norm_f32(const float* x, const float* w, float* y, long long rows, long long d, float eps)
{
	auto xt = make(x, { rows, d });
	auto wt = make(w, { d });
	auto yt = tensor_rms_norm<float32>(xt, -1, wt, eps);
	std::memcpy(y, yt.buffer(), sizeof(float) * rows * d);
}

}  // extern "C"
