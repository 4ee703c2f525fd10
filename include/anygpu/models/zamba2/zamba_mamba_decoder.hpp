// The Mamba half of a Zamba2 hybrid block: input RMSNorm, Mamba2 mixer, residual stream.
//   y = hidden_states + mixer(rms_norm(hidden_states, input_rmsnorm_weight, rms_norm_eps))
// Written in the style of the attention half, tensor_zamba_attention_decoder (anyGPU srcs/models/zamba2/zamba_attn_decoder.hpp:12-118:
// a weights struct that nests the block's weights and its norm weight, load_weights(paths...), a free function taking weights,
// cache, hidden states and the norm epsilon). One library call per invocation; the residual is added inside the last projection.
#pragma once

#include "zamba_mamba2_mixer.hpp"

template <typename dtype>
struct ZambaMambaDecoderweights
{
	ZambaMamba2weights<dtype> mixer_weights;
	Tensor<dtype, CUDA> input_rmsnorm_weight;  // (d_model)

	void load_weights(const std::string& md_path_in_rmsnorm_weight, const std::string& in_proj_path, const std::string& conv1d_weight_path,
		const std::string& conv1d_bias_path, const std::string& dt_bias_path, const std::string& A_log_path, const std::string& D_path,
		const std::string& norm_weight_path, const std::string& out_proj_path)
	{
		mixer_weights.load_weights(in_proj_path, conv1d_weight_path, conv1d_bias_path, dt_bias_path, A_log_path, D_path, norm_weight_path,
			out_proj_path);
		input_rmsnorm_weight = ZambaMamba2weights<dtype>::to_device(load_tensor<float32>(md_path_in_rmsnorm_weight));
	}
};

// hidden_states (batch, seq_len, d_model): prefill, the cache receives the states for decoding; (batch, d_model): one decode step.
template <typename dtype>
inline Tensor<dtype, CUDA> tensor_zamba_mamba_decoder(const ZambaMambaDecoderweights<dtype>& md_weights, ZambaMambaCache<dtype>& cache,
	const Tensor<dtype, CUDA>& hidden_states, const ZambaMamba2Config& config, const dtype rms_norm_eps)
{
	ACASSERT(hidden_states.dim == 3 || hidden_states.dim == 2, "hidden_states is (batch, seq_len, d_model) or (batch, d_model)");
	ACASSERT(hidden_states.shape[hidden_states.dim - 1] == config.d_model, "hidden size does not match the config");
	ACASSERT(md_weights.input_rmsnorm_weight.shape[0] == config.d_model, "input norm weight does not match the config");
	const b200_mamba2_config cfg = config.c_struct();
	const b200_mamba2_weights w = md_weights.mixer_weights.c_struct();
	const int dt = b200_dtype_of<dtype>();
	float e;
	if constexpr (std::is_same_v<dtype, float16>) e = __half2float(rms_norm_eps);
	else e = static_cast<float>(rms_norm_eps);
	Tensor<dtype, CUDA> out(hidden_states.dim, hidden_states.shape);
	const int64 batch = hidden_states.shape[0];
	if (hidden_states.dim == 3)
	{
		const int64 seqlen = hidden_states.shape[1];
		const size_t ws_bytes = b200_mamba2_decoder_prefill_workspace_bytes(&cfg, dt, batch, seqlen);
		void* ws = b200_workspace(ws_bytes);
		b200_check(b200_mamba2_decoder_prefill(dt, &cfg, &w, md_weights.input_rmsnorm_weight.buffer(), e, hidden_states.buffer(), out.buffer(),
			batch, seqlen, nullptr, cache.conv_state.buffer(), cache.ssm_state.buffer(), ws, ws_bytes, nullptr),
			"tensor_zamba_mamba_decoder (prefill)");
	}
	else
	{
		const size_t ws_bytes = b200_mamba2_decoder_decode_workspace_bytes(&cfg, dt, batch);
		void* ws = b200_workspace(ws_bytes);
		b200_check(b200_mamba2_decoder_decode(dt, &cfg, &w, md_weights.input_rmsnorm_weight.buffer(), e, hidden_states.buffer(), out.buffer(),
			cache.conv_state.buffer(), cache.ssm_state.buffer(), batch, ws, ws_bytes, nullptr), "tensor_zamba_mamba_decoder (decode)");
	}
	return out;
}
