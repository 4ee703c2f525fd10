// The Mamba2 mixer of a Zamba2 block as a model-level operator: weights struct with load_weights(paths...), cache struct,
// config struct and a tensor_zamba_<block>(weights, cache, hidden_states, config) free function, in the style of anyGPU's other
// Zamba2 blocks (weights + load_weights: srcs/models/zamba2/zamba_mlp.hpp:13-48; block function with cache and config
// arguments: srcs/models/zamba2/zamba_attn_decoder.hpp:68-118). anyGPU itself lists this layer as not yet written
// (docs/TODO_backlog.md:3-25); ZambaMambaCache fills the role of its empty ZambaKVcache (zamba_sdpa.hpp:13).
#pragma once

#include "../../b200_call.hpp"
#include "../../io/dat_file.hpp"
#include "../../io/safetensors_file.hpp"

struct ZambaMamba2Config
{
	int64 d_model = 2048, d_inner = 4096, nheads = 64, headdim = 64, d_state = 64, ngroups = 1, d_conv = 4, chunk = 256;
	int64 norm_group_size = 0;  // 0: the gated RMSNorm statistic spans the whole row (anyGPU's behaviour)
	float eps = 1e-5f;

	int64 conv_dim() const { return d_inner + 2 * ngroups * d_state; }
	int64 d_in_proj() const { return 2 * d_inner + 2 * ngroups * d_state + nheads; }
	b200_mamba2_config c_struct() const { return { d_model, d_inner, nheads, headdim, d_state, ngroups, d_conv, chunk, norm_group_size, eps }; }
};

template <typename dtype>
struct ZambaMamba2weights
{
	Tensor<dtype, CUDA> in_proj_weight;   // (d_model, d_in_proj): (in_features, out_features), what tensor_linear takes
	Tensor<dtype, CUDA> conv1d_weight;    // (conv_dim, d_conv)
	Tensor<dtype, CUDA> conv1d_bias;      // (conv_dim)
	Tensor<float32, CUDA> dt_bias;        // (nheads)
	Tensor<float32, CUDA> A_log;          // (nheads)
	Tensor<float32, CUDA> D;              // (nheads)
	Tensor<dtype, CUDA> norm_weight;      // (d_inner)
	Tensor<dtype, CUDA> out_proj_weight;  // (d_inner, d_model)

	// Loads float32 .dat dumps of a checkpoint's mamba.{in_proj,conv1d,dt_bias,A_log,D,norm,out_proj} tensors. Projection
	// weights are stored (out_features, in_features) in checkpoints and are transposed here, at load time, exactly as
	// anyGPU does for its other Zamba2 linear layers (srcs/models/zamba2/zamba_mlp.hpp:26-29). conv1d.weight may be
	// (conv_dim, 1, d_conv) or (conv_dim, d_conv).
	void load_weights(const std::string& in_proj_path, const std::string& conv1d_weight_path, const std::string& conv1d_bias_path,
		const std::string& dt_bias_path, const std::string& A_log_path, const std::string& D_path, const std::string& norm_weight_path,
		const std::string& out_proj_path)
	{
		in_proj_weight = to_device(transposed(load_tensor<float32>(in_proj_path)));
		auto cw = load_tensor<float32>(conv1d_weight_path);
		if (cw.dim == 3) cw = tensor_view(cw, { cw.shape[0], cw.shape[2] });
		conv1d_weight = to_device(cw);
		conv1d_bias = to_device(load_tensor<float32>(conv1d_bias_path));
		dt_bias = load_tensor<float32>(dt_bias_path).copy_to_cuda();
		A_log = load_tensor<float32>(A_log_path).copy_to_cuda();
		D = load_tensor<float32>(D_path).copy_to_cuda();
		norm_weight = to_device(load_tensor<float32>(norm_weight_path));
		out_proj_weight = to_device(transposed(load_tensor<float32>(out_proj_path)));
	}

	// The same tensors straight from a .safetensors checkpoint: `prefix` + {in_proj.weight, conv1d.weight, conv1d.bias, dt_bias,
	// A_log, D, norm.weight, out_proj.weight}, e.g. prefix "model.layers.3.mamba." (stored F32, F16 or BF16).
	void load_safetensors(const std::string& path, const std::string& prefix)
	{
		auto get = [&](const char* leaf) { return sft_read_tensor_f32(path, prefix + leaf); };
		in_proj_weight = to_device(transposed(get("in_proj.weight")));
		auto cw = get("conv1d.weight");
		if (cw.dim == 3) cw = tensor_view(cw, { cw.shape[0], cw.shape[2] });
		conv1d_weight = to_device(cw);
		conv1d_bias = to_device(get("conv1d.bias"));
		dt_bias = get("dt_bias").copy_to_cuda();
		A_log = get("A_log").copy_to_cuda();
		D = get("D").copy_to_cuda();
		norm_weight = to_device(get("norm.weight"));
		out_proj_weight = to_device(transposed(get("out_proj.weight")));
	}

	b200_mamba2_weights c_struct() const
	{
		return { in_proj_weight.buffer(), conv1d_weight.buffer(), conv1d_bias.buffer(), dt_bias.buffer(), A_log.buffer(), D.buffer(),
			norm_weight.buffer(), out_proj_weight.buffer(), B200_W_KN, B200_W_KN };
	}

	static Tensor<dtype, CUDA> to_device(const Tensor<float32, CPU>& t)
	{
		if constexpr (std::is_same_v<dtype, float32>) return t.copy_to_cuda();
		else return cvt_tensor_datatype<dtype, float32>(t).copy_to_cuda();
	}

private:
	static Tensor<float32, CPU> transposed(const Tensor<float32, CPU>& t)
	{
		const int64 r = t.shape[0], c = t.shape[1];
		Tensor<float32, CPU> out(std::vector<int64>{ c, r });
		for (int64 i = 0; i < r; ++i)
			for (int64 j = 0; j < c; ++j) out.buffer()[j * r + i] = t.buffer()[i * c + j];
		return out;
	}
};

template <typename dtype>
struct ZambaMambaCache
{
	Tensor<dtype, CUDA> conv_state;     // (batch, conv_dim, d_conv - 1), oldest input first
	Tensor<float32, CUDA> ssm_state;    // (batch, nheads, headdim, d_state)

	ZambaMambaCache() = default;
	ZambaMambaCache(const ZambaMamba2Config& cfg, const int64 batch)
		: conv_state(std::vector<int64>{ batch, cfg.conv_dim(), cfg.d_conv - 1 }),
		  ssm_state(std::vector<int64>{ batch, cfg.nheads, cfg.headdim, cfg.d_state })
	{
		CUDA_CHECK(cudaMemset(conv_state.raw_buffer(), 0, static_cast<size_t>(conv_state.capacity())));
		CUDA_CHECK(cudaMemset(ssm_state.raw_buffer(), 0, static_cast<size_t>(ssm_state.capacity())));
	}
};

// hidden_states (batch, seq_len, d_model): prefill of the whole sequence; the cache receives the conv and SSM states that
// a following decode step needs. hidden_states (batch, d_model): one decode step, cache advanced in place.
template <typename dtype>
inline Tensor<dtype, CUDA> tensor_zamba_mamba2_mixer(const ZambaMamba2weights<dtype>& weights, ZambaMambaCache<dtype>& cache,
	const Tensor<dtype, CUDA>& hidden_states, const ZambaMamba2Config& config)
{
	ACASSERT(hidden_states.dim == 3 || hidden_states.dim == 2, "hidden_states is (batch, seq_len, d_model) or (batch, d_model)");
	ACASSERT(hidden_states.shape[hidden_states.dim - 1] == config.d_model, "hidden size does not match the config");
	const b200_mamba2_config cfg = config.c_struct();
	const b200_mamba2_weights w = weights.c_struct();
	const int dt = b200_dtype_of<dtype>();
	Tensor<dtype, CUDA> out(hidden_states.dim, hidden_states.shape);
	const int64 batch = hidden_states.shape[0];
	if (hidden_states.dim == 3)
	{
		const int64 seqlen = hidden_states.shape[1];
		const size_t ws_bytes = b200_mamba2_mixer_prefill_workspace_bytes(&cfg, dt, batch, seqlen);
		void* ws = b200_workspace(ws_bytes);
		b200_check(b200_mamba2_mixer_prefill(dt, &cfg, &w, hidden_states.buffer(), out.buffer(), batch, seqlen, nullptr,
			cache.conv_state.buffer(), cache.ssm_state.buffer(), ws, ws_bytes, nullptr), "tensor_zamba_mamba2_mixer (prefill)");
	}
	else
	{
		const size_t ws_bytes = b200_mamba2_mixer_decode_workspace_bytes(&cfg, dt, batch);
		void* ws = b200_workspace(ws_bytes);
		b200_check(b200_mamba2_mixer_decode(dt, &cfg, &w, hidden_states.buffer(), out.buffer(), cache.conv_state.buffer(),
			cache.ssm_state.buffer(), batch, ws, ws_bytes, nullptr), "tensor_zamba_mamba2_mixer (decode)");
	}
	return out;
}

// The next tokens (batch, seq_len, d_model) of sequences whose state so far is in `cache` (a freshly constructed cache for new
// sequences): chunked prefill of long prompts. Any split of a prompt into pieces gives the outputs and the cache of one call.
template <typename dtype>
inline Tensor<dtype, CUDA> tensor_zamba_mamba2_mixer_continue(const ZambaMamba2weights<dtype>& weights, ZambaMambaCache<dtype>& cache,
	const Tensor<dtype, CUDA>& hidden_states, const ZambaMamba2Config& config)
{
	ACASSERT(hidden_states.dim == 3, "hidden_states is (batch, seq_len, d_model)");
	ACASSERT(hidden_states.shape[2] == config.d_model, "hidden size does not match the config");
	const b200_mamba2_config cfg = config.c_struct();
	const b200_mamba2_weights w = weights.c_struct();
	const int dt = b200_dtype_of<dtype>();
	Tensor<dtype, CUDA> out(hidden_states.dim, hidden_states.shape);
	const int64 batch = hidden_states.shape[0], seqlen = hidden_states.shape[1];
	const size_t ws_bytes = b200_mamba2_mixer_prefill_continue_workspace_bytes(&cfg, dt, batch, seqlen);
	void* ws = b200_workspace(ws_bytes);
	b200_check(b200_mamba2_mixer_prefill_continue(dt, &cfg, &w, hidden_states.buffer(), out.buffer(), batch, seqlen,
		cache.conv_state.buffer(), cache.ssm_state.buffer(), ws, ws_bytes, nullptr), "tensor_zamba_mamba2_mixer_continue");
	return out;
}

// A packed batch: hidden_states (total_tokens, d_model) holds cu_seqlens.size()-1 sequences back to back, sequence s in rows
// cu_seqlens[s] .. cu_seqlens[s+1]-1. `cache` (one entry per sequence) receives the final states. Every sequence gets what
// tensor_zamba_mamba2_mixer gives for it alone.
template <typename dtype>
inline Tensor<dtype, CUDA> tensor_zamba_mamba2_mixer_varlen(const ZambaMamba2weights<dtype>& weights, ZambaMambaCache<dtype>& cache,
	const Tensor<dtype, CUDA>& hidden_states, const std::vector<int64>& cu_seqlens, const ZambaMamba2Config& config)
{
	ACASSERT(hidden_states.dim == 2, "hidden_states is (total_tokens, d_model)");
	ACASSERT(hidden_states.shape[1] == config.d_model, "hidden size does not match the config");
	ACASSERT(!cu_seqlens.empty() && cu_seqlens.back() == hidden_states.shape[0], "cu_seqlens must end at the token count");
	const int64 nseq = static_cast<int64>(cu_seqlens.size()) - 1;
	ACASSERT(cache.conv_state.shape[0] == nseq && cache.ssm_state.shape[0] == nseq, "one cache entry per sequence");
	const b200_mamba2_config cfg = config.c_struct();
	const b200_mamba2_weights w = weights.c_struct();
	const int dt = b200_dtype_of<dtype>();
	Tensor<dtype, CUDA> out(hidden_states.dim, hidden_states.shape);
	const size_t ws_bytes = b200_mamba2_mixer_prefill_varlen_workspace_bytes(&cfg, dt, hidden_states.shape[0]);
	void* ws = b200_workspace(ws_bytes);
	static_assert(sizeof(int64) == sizeof(int64_t), "cu_seqlens is passed as int64_t");
	b200_check(b200_mamba2_mixer_prefill_varlen(dt, &cfg, &w, hidden_states.buffer(), out.buffer(),
		reinterpret_cast<const int64_t*>(cu_seqlens.data()), nseq, nullptr, cache.conv_state.buffer(), cache.ssm_state.buffer(), ws, ws_bytes,
		nullptr), "tensor_zamba_mamba2_mixer_varlen");
	return out;
}
