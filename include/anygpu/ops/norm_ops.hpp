// tensor_rms_norm for CUDA tensors, float16 and float32. Same signature as anyGPU srcs/ops/norm_ops.hpp:196-228 (whose CUDA
// overload accepts float32 only); the norm region is the last axis, which is every use on the Zamba2 path (axis = -1).
#pragma once

#include "../b200_call.hpp"

template <typename dtype>
inline Tensor<dtype, CUDA> tensor_rms_norm(const Tensor<dtype, CUDA>& xt, const int32 axis, const Tensor<dtype, CUDA> wt, const dtype eps,
	const bool zero_centered = false)
{
	const int32 dim = xt.dim;
	ACASSERT((-dim <= axis && axis < dim), "axis is out of range");
	ACASSERT((dim + axis) % dim == dim - 1, "the norm region is the last axis");
	const int64 d = xt.shape[dim - 1];
	ACASSERT(wt.shape[0] == d, "wt shape is incorrect");
	Tensor<dtype, CUDA> yt(dim, xt.shape);
	const int64 xs = dim >= 2 ? xt.stride[dim - 2] : d;
	float e;
	if constexpr (std::is_same_v<dtype, float16>) e = __half2float(eps);
	else e = static_cast<float>(eps);
	b200_check(b200_rms_norm(b200_dtype_of<dtype>(), xt.buffer(), xs, wt.buffer(), yt.buffer(), d, xt.numel() / d, d, e, zero_centered ? 1 : 0,
		nullptr), "tensor_rms_norm");
	return yt;
}
