// tensor_causal_conv1d for CUDA tensors (float16 and float32) and the decode-step update.
// Same contract as anyGPU srcs/fused/causal_conv1d.hpp:90-117: xt (batch, dims, seq_len), wt (dims, width <= 4), bt (dims)
// -> silu(conv1d(x, w.unsqueeze(1), b, padding=width-1, groups=dims))[..., :seq_len]. The reference's CUDA overload is
// float32-only; here float16 is the main path (fp32 accumulation).
#pragma once

#include "../b200_call.hpp"

template <typename dtype>
inline Tensor<dtype, CUDA> tensor_causal_conv1d(const Tensor<dtype, CUDA>& xt, const Tensor<dtype, CUDA>& wt, const Tensor<dtype, CUDA>& bt)
{
	ACASSERT(xt.dim == 3, "xt needs to be 3 dimensional");
	ACASSERT(xt.shape[1] == wt.shape[0], "xt and wt need to have the same dims");
	ACASSERT(wt.shape[0] == bt.shape[0], "wt and bt need to have the same dims");
	ACASSERT(wt.shape[1] <= 4, "kernel width needs to be under 4");
	Tensor<dtype, CUDA> yt(xt.dim, xt.shape);
	b200_check(b200_causal_conv1d(b200_dtype_of<dtype>(), xt.buffer(), wt.buffer(), bt.buffer(), yt.buffer(), xt.shape[0], xt.shape[1],
		xt.shape[2], static_cast<int>(wt.shape[1]), nullptr), "tensor_causal_conv1d");
	return yt;
}

// One decode step. x_t (batch, dims); conv_state (batch, dims, width-1), oldest input first, advanced IN PLACE.
// Step t returns column t of tensor_causal_conv1d applied to the whole history.
template <typename dtype>
inline Tensor<dtype, CUDA> tensor_causal_conv1d_update(const Tensor<dtype, CUDA>& x_t, Tensor<dtype, CUDA>& conv_state,
	const Tensor<dtype, CUDA>& wt, const Tensor<dtype, CUDA>& bt)
{
	ACASSERT(x_t.dim == 2 && conv_state.dim == 3, "x_t is (batch, dims), conv_state is (batch, dims, width-1)");
	ACASSERT(conv_state.shape[2] == wt.shape[1] - 1, "conv_state holds width-1 inputs");
	Tensor<dtype, CUDA> y_t(x_t.dim, x_t.shape);
	b200_check(b200_causal_conv1d_update(b200_dtype_of<dtype>(), x_t.buffer(), x_t.stride[0], conv_state.buffer(), wt.buffer(), bt.buffer(),
		y_t.buffer(), y_t.stride[0], x_t.shape[0], x_t.shape[1], static_cast<int>(wt.shape[1]), nullptr), "tensor_causal_conv1d_update");
	return y_t;
}
