// SSD chunked selective scan and its single-token form as tensor operators. anyGPU has this computation only as a
// PyTorch script; names and argument order follow mamba_chunk_scan_combined_ref
// (scripts/zamba2/mamba_chunk_scan_comb.py:167-172): x (b,l,H,P), dt (b,l,H), A (H), B/C (b,l,G,N), chunk_size,
// D (H), dt_bias (H), initial_states (b,H,P,N); dt_softplus is always on. A, D, dt_bias and all states are float32.
#pragma once

#include "../b200_call.hpp"

template <typename dtype>
struct MambaChunkScanResult
{
	Tensor<dtype, CUDA> y;                  // (b, l, H, P)
	Tensor<float32, CUDA> final_states;     // (b, H, P, N)
};

template <typename dtype>
inline MambaChunkScanResult<dtype> tensor_mamba_chunk_scan_combined(const Tensor<dtype, CUDA>& x, const Tensor<dtype, CUDA>& dt,
	const Tensor<float32, CUDA>& A, const Tensor<dtype, CUDA>& B, const Tensor<dtype, CUDA>& C, const int64 chunk_size,
	const Tensor<float32, CUDA>* D = nullptr, const Tensor<float32, CUDA>* dt_bias = nullptr,
	const Tensor<float32, CUDA>* initial_states = nullptr)
{
	ACASSERT(x.dim == 4 && dt.dim == 3 && B.dim == 4 && C.dim == 4, "x (b,l,H,P), dt (b,l,H), B/C (b,l,G,N)");
	const int64 b = x.shape[0], l = x.shape[1], H = x.shape[2], P = x.shape[3], G = B.shape[2], N = B.shape[3];
	ACASSERT(H % G == 0 && dt.shape[2] == H && A.shape[0] == H, "head / group counts do not match");
	MambaChunkScanResult<dtype> r{ Tensor<dtype, CUDA>(x.dim, x.shape), Tensor<float32, CUDA>(std::vector<int64>{ b, H, P, N }) };
	const size_t ws_bytes = b200_mamba_chunk_scan_combined_workspace_bytes(b, l, H, P, G, N, chunk_size);
	void* ws = b200_workspace(ws_bytes);
	b200_check(b200_mamba_chunk_scan_combined(b200_dtype_of<dtype>(), x.buffer(), x.stride[1], dt.buffer(), dt.stride[1], A.buffer(), 0,
		B.buffer(), B.stride[1], C.buffer(), C.stride[1], D ? D->buffer() : nullptr, dt_bias ? dt_bias->buffer() : nullptr,
		initial_states ? initial_states->buffer() : nullptr, r.y.buffer(), H * P, r.final_states.buffer(), b, l, H, P, G, N, chunk_size, 1,
		ws, ws_bytes, nullptr), "tensor_mamba_chunk_scan_combined");
	return r;
}

// One decode step: ssm_state (b,H,P,N) float32 advanced IN PLACE; x (b,H,P), dt (b,H), B/C (b,G,N) -> y (b,H,P).
template <typename dtype>
inline Tensor<dtype, CUDA> tensor_mamba_selective_state_update(Tensor<float32, CUDA>& ssm_state, const Tensor<dtype, CUDA>& x,
	const Tensor<dtype, CUDA>& dt, const Tensor<float32, CUDA>& A, const Tensor<dtype, CUDA>& B, const Tensor<dtype, CUDA>& C,
	const Tensor<float32, CUDA>* D = nullptr, const Tensor<float32, CUDA>* dt_bias = nullptr)
{
	ACASSERT(x.dim == 3 && dt.dim == 2 && B.dim == 3, "x (b,H,P), dt (b,H), B/C (b,G,N)");
	const int64 b = x.shape[0], H = x.shape[1], P = x.shape[2], G = B.shape[1], N = B.shape[2];
	Tensor<dtype, CUDA> y(x.dim, x.shape);
	b200_check(b200_selective_state_update(b200_dtype_of<dtype>(), ssm_state.buffer(), x.buffer(), x.stride[0], dt.buffer(), dt.stride[0],
		A.buffer(), 0, B.buffer(), B.stride[0], C.buffer(), C.stride[0], D ? D->buffer() : nullptr, dt_bias ? dt_bias->buffer() : nullptr,
		y.buffer(), H * P, b, H, P, G, N, 1, nullptr), "tensor_mamba_selective_state_update");
	return y;
}
