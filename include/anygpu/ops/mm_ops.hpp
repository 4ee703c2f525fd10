// tensor_mm / tensor_linear for CUDA tensors on top of b200_linear. Same names, argument meaning and result shapes as
// anyGPU srcs/ops/mm_ops.hpp:48-97 (tensor_mm, 3- and 2-argument) and :206-232 (tensor_linear without bias);
// weights are (in_features, out_features). float16 runs on the tcgen05 kernel (fp32 accumulation, any M; K and N
// multiples of 8), float32 on the exact SIMT kernel.
#pragma once

#include "../b200_call.hpp"

template <typename dtype>
inline void tensor_mm(const Tensor<dtype, CUDA>& lhs, const Tensor<dtype, CUDA>& rhs, Tensor<dtype, CUDA>& res)
{
	ACASSERT(lhs.dim == 2 && rhs.dim == 2 && lhs.shape[1] == rhs.shape[0], "matrix multiplication requires compatible matrices");
	ACASSERT(lhs.shape[0] == res.shape[0] && rhs.shape[1] == res.shape[1], "result mtx shape is wrong");
	ACASSERT(rhs.stride[1] == 1 && rhs.stride[0] == rhs.shape[1], "rhs must be dense row-major");
	b200_check(b200_linear(b200_dtype_of<dtype>(), lhs.buffer(), lhs.stride[0], rhs.buffer(), B200_W_KN, res.buffer(), res.stride[0],
		lhs.shape[0], lhs.shape[1], rhs.shape[1], nullptr), "tensor_mm");
}

template <typename dtype>
inline Tensor<dtype, CUDA> tensor_mm(const Tensor<dtype, CUDA>& lhs, const Tensor<dtype, CUDA>& rhs)
{
	Tensor<dtype, CUDA> res(std::vector<int64>{ lhs.shape[0], rhs.shape[1] });
	tensor_mm(lhs, rhs, res);
	return res;
}

template <typename dtype>
inline Tensor<dtype, CUDA> tensor_linear(const Tensor<dtype, CUDA>& xt,  // (*, in_features)
	const Tensor<dtype, CUDA>& wt)                                      // (in_features, out_features)
{
	const int64 d = xt.dim;
	const int64 cols = xt.shape[d - 1];
	const int64 rows = xt.numel() / cols;
	ACASSERT(cols == wt.shape[0], "xt and wt need matching in_features");
	std::vector<int64> y_shape(static_cast<size_t>(d));
	for (int64 i = 0; i < d - 1; ++i) y_shape[static_cast<size_t>(i)] = xt.shape[i];
	y_shape[static_cast<size_t>(d - 1)] = wt.shape[1];
	Tensor<dtype, CUDA> y(y_shape);
	// rows of xt may be strided (a last-axis slice view): the row stride is the stride of the second-to-last axis
	const int64 ldx = d >= 2 ? xt.stride[d - 2] : cols;
	b200_check(b200_linear(b200_dtype_of<dtype>(), xt.buffer(), ldx, wt.buffer(), B200_W_KN, y.buffer(), wt.shape[1], rows, cols,
		wt.shape[1], nullptr), "tensor_linear");
	return y;
}
