// tensor_zamba_gated_rmsnorm for CUDA tensors: one fused kernel instead of silu -> mul -> rms_norm.
// Same signature as anyGPU srcs/models/zamba2/zamba_gated_rmsnorm.hpp:9-23. Like the reference, the statistic spans
// the whole last axis and `gsize` is ignored (its own comment: "the gated mechanism is not implemented here ... fallback to
// the normal case"); tensor_zamba_gated_rmsnorm_grouped honours the group size.
#pragma once

#include "../../b200_call.hpp"

template <typename dtype>
inline Tensor<dtype, CUDA> tensor_zamba_gated_rmsnorm_grouped(const Tensor<dtype, CUDA>& xt, const Tensor<dtype, CUDA>& zt,
	const Tensor<dtype, CUDA>& wt, const int64 group_size, const dtype eps)
{
	const int64 d = xt.shape[xt.dim - 1];
	ACASSERT(zt.shape[zt.dim - 1] == d && wt.shape[0] == d, "x, z and w need the same last axis");
	Tensor<dtype, CUDA> yt(xt.dim, xt.shape);
	const int64 xs = xt.dim >= 2 ? xt.stride[xt.dim - 2] : d;
	const int64 zs = zt.dim >= 2 ? zt.stride[zt.dim - 2] : d;
	float e;
	if constexpr (std::is_same_v<dtype, float16>) e = __half2float(eps);
	else e = static_cast<float>(eps);
	b200_check(b200_gated_rmsnorm(b200_dtype_of<dtype>(), xt.buffer(), xs, zt.buffer(), zs, wt.buffer(), yt.buffer(), d, xt.numel() / d, d,
		group_size, e, nullptr), "tensor_zamba_gated_rmsnorm");
	return yt;
}

template <typename dtype>
inline Tensor<dtype, CUDA> tensor_zamba_gated_rmsnorm(const Tensor<dtype, CUDA>& xt, const Tensor<dtype, CUDA>& zt,
	const Tensor<dtype, CUDA>& wt, const int gsize, const dtype eps)
{
	(void)gsize;  // ignored, as in the reference
	return tensor_zamba_gated_rmsnorm_grouped(xt, zt, wt, xt.shape[xt.dim - 1], eps);
}
