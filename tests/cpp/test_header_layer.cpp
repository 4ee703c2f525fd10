// Exercises the C++ header layer (include/anygpu) on a GPU against the CPU oracle, in the style of anyGPU's own tests
// (tests/tests.cpp: run the CUDA overload, copy to host, compare with the CPU reference, print
// "TestCase [name - CUDA]: PASSED|FAILED"). Unlike those, the process exit code reports failure.
// Links libanygpu_b200.so (the product) and liboracle.so (test infrastructure, the checker).
#include <cmath>
#include <cstdio>
#include <cstring>
#include <fstream>

#include "anygpu/fused/causal_conv1d.hpp"
#include "anygpu/fused/mamba_chunk_scan.hpp"
#include "anygpu/models/zamba2/zamba_gated_rmsnorm.hpp"
#include "anygpu/models/zamba2/zamba_mamba2_mixer.hpp"
#include "anygpu/models/zamba2/zamba_mamba_decoder.hpp"
#include "anygpu/ops/norm_ops.hpp"
#include "anygpu/ops/mm_ops.hpp"

extern "C" {
void orc_linear_f32_fast(const float*, const float*, float*, int64_t, int64_t, int64_t);
void orc_causal_conv1d_f32(const float*, const float*, const float*, float*, int64_t, int64_t, int64_t, int64_t);
void orc_causal_conv1d_update_f32(const float*, float*, const float*, const float*, float*, int64_t, int64_t, int64_t);
void orc_gated_rmsnorm_f32(const float*, const float*, const float*, float*, int64_t, int64_t, int64_t, float);
void orc_rms_norm_f32(const float*, const float*, float*, int64_t, int64_t, float, int);
void orc_ssd_chunk_scan_f32(const float*, const float*, const float*, const float*, const float*, const float*, const float*,
	const float*, float*, float*, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int);
void orc_mamba2_mixer_prefill_f32(const float*, const float*, const float*, const float*, const float*, const float*, const float*,
	const float*, const float*, const float*, float*, float*, float*, float*, float*, float*, float*, int64_t, int64_t, int64_t,
	int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, float, int);
void orc_mamba2_mixer_decode_f32(const float*, const float*, const float*, const float*, const float*, const float*, const float*,
	const float*, const float*, float*, float*, float*, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t,
	int64_t, float, int);
}

static int g_failed = 0;

// element passes if |a-e| <= abs_tol OR |a-e| <= rel_tol * |e|
template <typename T>
static bool close_enough(const Tensor<T, CPU>& actual, const std::vector<float>& expected, float rel_tol, float abs_tol, double max_bad_fraction = 0.0)
{
	const int64 n = actual.numel();
	if (static_cast<size_t>(n) != expected.size()) return false;
	int64 bad = 0;
	for (int64 i = 0; i < n; ++i)
	{
		float a;
		if constexpr (std::is_same_v<T, float16>) a = __half2float(actual.buffer()[i]);
		else a = actual.buffer()[i];
		const float err = std::fabs(a - expected[static_cast<size_t>(i)]);
		if (!(err <= abs_tol || err <= rel_tol * std::fabs(expected[static_cast<size_t>(i)]))) ++bad;
	}
	return static_cast<double>(bad) <= max_bad_fraction * static_cast<double>(n);
}

static void report(const char* name, bool ok)
{
	std::printf("TestCase [%s - CUDA]: %s\n", name, ok ? "PASSED" : "FAILED");
	if (!ok) ++g_failed;
}

static std::vector<float> host_f32(const Tensor<float16, CPU>& t)
{
	std::vector<float> v(static_cast<size_t>(t.numel()));
	for (size_t i = 0; i < v.size(); ++i) v[i] = __half2float(t.buffer()[i]);
	return v;
}
static std::vector<float> host_f32(const Tensor<float32, CPU>& t)
{
	return std::vector<float>(t.buffer(), t.buffer() + t.numel());
}

static void test_causal_conv1d_f16()
{
	const int64 b = 2, d = 48, s = 128, w = 4;
	auto hx = cvt_tensor_datatype<float16, float32>(crt_random_normal_tensor<float32, CPU>({ b, d, s }, 1));
	auto hw = cvt_tensor_datatype<float16, float32>(crt_random_normal_tensor<float32, CPU>({ d, w }, 2, 0.5f));
	auto hb = cvt_tensor_datatype<float16, float32>(crt_random_normal_tensor<float32, CPU>({ d }, 3, 0.1f));
	auto y = tensor_causal_conv1d(hx.copy_to_cuda(), hw.copy_to_cuda(), hb.copy_to_cuda()).copy_to_host();
	std::vector<float> fx = host_f32(hx), fw = host_f32(hw), fb = host_f32(hb), e(fx.size());
	orc_causal_conv1d_f32(fx.data(), fw.data(), fb.data(), e.data(), b, d, s, w);
	report("tensor_causal_conv1d f16", close_enough(y, e, 2e-2f, 2e-3f));

	// decode steps reproduce the columns of the full-sequence result
	Tensor<float16, CUDA> state(std::vector<int64>{ b, d, w - 1 });
	CUDA_CHECK(cudaMemset(state.raw_buffer(), 0, static_cast<size_t>(state.capacity())));
	auto dw = hw.copy_to_cuda(), db = hb.copy_to_cuda();
	bool ok = true;
	for (int64 t = 0; t < 6 && ok; ++t)
	{
		Tensor<float16, CPU> col(std::vector<int64>{ b, d });
		std::vector<float> ecol(static_cast<size_t>(b * d));
		for (int64 i = 0; i < b * d; ++i)
		{
			col.buffer()[i] = hx.buffer()[i * s + t];
			ecol[static_cast<size_t>(i)] = e[static_cast<size_t>(i * s + t)];
		}
		auto yt = tensor_causal_conv1d_update(col.copy_to_cuda(), state, dw, db).copy_to_host();
		ok = close_enough(yt, ecol, 2e-2f, 2e-3f);
	}
	report("tensor_causal_conv1d_update f16", ok);
}

static void test_linear_f16()
{
	const int64 m = 200, k = 264, n = 1064;
	auto hx = cvt_tensor_datatype<float16, float32>(crt_random_normal_tensor<float32, CPU>({ 2, m / 2, k }, 4));
	auto hw = cvt_tensor_datatype<float16, float32>(crt_random_normal_tensor<float32, CPU>({ k, n }, 5, 0.05f));
	auto y = tensor_linear(hx.copy_to_cuda(), hw.copy_to_cuda());
	bool ok = y.dim == 3 && y.shape[0] == 2 && y.shape[1] == m / 2 && y.shape[2] == n;
	std::vector<float> fx = host_f32(hx), fw = host_f32(hw), e(static_cast<size_t>(m * n));
	orc_linear_f32_fast(fx.data(), fw.data(), e.data(), m, k, n);
	report("tensor_linear f16", ok && close_enough(y.copy_to_host(), e, 2e-2f, 2e-3f));
}

static void test_gated_rmsnorm_f32()
{
	const int64 rows = 6, d = 512;
	auto hx = crt_random_normal_tensor<float32, CPU>({ 2, 3, d }, 6);
	auto hz = crt_random_normal_tensor<float32, CPU>({ 2, 3, d }, 7);
	auto hw = crt_random_normal_tensor<float32, CPU>({ d }, 8);
	auto y = tensor_zamba_gated_rmsnorm(hx.copy_to_cuda(), hz.copy_to_cuda(), hw.copy_to_cuda(), 4096, 1e-5f).copy_to_host();
	std::vector<float> e(static_cast<size_t>(rows * d));
	orc_gated_rmsnorm_f32(hx.buffer(), hz.buffer(), hw.buffer(), e.data(), rows, d, d, 1e-5f);
	report("tensor_zamba_gated_rmsnorm f32", close_enough(y, e, 0.f, 1e-3f));  // anyGPU's rule for this op: abs 1e-3
}

static void test_chunk_scan_f16()
{
	const int64 b = 1, l = 512, H = 4, P = 64, G = 1, N = 64, Q = 256;
	auto hx = cvt_tensor_datatype<float16, float32>(crt_random_normal_tensor<float32, CPU>({ b, l, H, P }, 9, 0.5f));
	auto hdt = cvt_tensor_datatype<float16, float32>(crt_random_normal_tensor<float32, CPU>({ b, l, H }, 10));
	auto hB = cvt_tensor_datatype<float16, float32>(crt_random_normal_tensor<float32, CPU>({ b, l, G, N }, 11, 0.5f));
	auto hC = cvt_tensor_datatype<float16, float32>(crt_random_normal_tensor<float32, CPU>({ b, l, G, N }, 12, 0.5f));
	Tensor<float32, CPU> hA(std::vector<int64>{ H }), hD(std::vector<int64>{ H }), hbias(std::vector<int64>{ H });
	for (int64 h = 0; h < H; ++h)
	{
		hA.buffer()[h] = -(1.0f + 3.5f * static_cast<float>(h));
		hD.buffer()[h] = 1.0f;
		hbias.buffer()[h] = -3.0f;
	}
	auto dD = hD.copy_to_cuda(), dbias = hbias.copy_to_cuda();
	auto r = tensor_mamba_chunk_scan_combined(hx.copy_to_cuda(), hdt.copy_to_cuda(), hA.copy_to_cuda(), hB.copy_to_cuda(), hC.copy_to_cuda(), Q,
		&dD, &dbias);
	std::vector<float> fx = host_f32(hx), fdt = host_f32(hdt), fB = host_f32(hB), fC = host_f32(hC), ey(fx.size()),
		efs(static_cast<size_t>(b * H * P * N));
	orc_ssd_chunk_scan_f32(fx.data(), fdt.data(), hA.buffer(), fB.data(), fC.data(), hD.buffer(), hbias.buffer(), nullptr, ey.data(),
		efs.data(), b, l, H, P, G, N, Q, 1);
	report("tensor_mamba_chunk_scan_combined f16 (y)", close_enough(r.y.copy_to_host(), ey, 2e-2f, 2e-3f));
	report("tensor_mamba_chunk_scan_combined f16 (final_states)", close_enough(r.final_states.copy_to_host(), efs, 2e-2f, 2e-3f));
}

static void test_rms_norm()
{
	const int64 rows = 6, d = 520;
	auto hx = crt_random_normal_tensor<float32, CPU>({ 2, 3, d }, 30);
	auto hw = crt_random_normal_tensor<float32, CPU>({ d }, 31);
	auto y = tensor_rms_norm(hx.copy_to_cuda(), -1, hw.copy_to_cuda(), 1e-5f).copy_to_host();
	std::vector<float> e(static_cast<size_t>(rows * d));
	orc_rms_norm_f32(hx.buffer(), hw.buffer(), e.data(), rows, d, 1e-5f, 0);
	report("tensor_rms_norm f32", close_enough(y, e, 0.f, 1e-3f));
	auto hx16 = cvt_tensor_datatype<float16, float32>(hx);
	auto hw16 = cvt_tensor_datatype<float16, float32>(hw);
	auto y16 = tensor_rms_norm(hx16.copy_to_cuda(), -1, hw16.copy_to_cuda(), __float2half(1e-5f), true);
	auto fx = host_f32(hx16);
	auto fw = host_f32(hw16);
	orc_rms_norm_f32(fx.data(), fw.data(), e.data(), rows, d, __half2float(__float2half(1e-5f)), 1);
	report("tensor_rms_norm f16 zero-centered", close_enough(y16.copy_to_host(), e, 2e-2f, 2e-3f));
}

static void test_mixer_f32_and_dat_files(const std::string& tmp_dir)
{
	// configuration-0 sizes: batch 1, seqlen 64, d_model 256, d_inner 512, 8 heads x 64, d_state 16, chunk 32
	ZambaMamba2Config cfg;
	cfg.d_model = 256; cfg.d_inner = 512; cfg.nheads = 8; cfg.headdim = 64; cfg.d_state = 16; cfg.ngroups = 1; cfg.d_conv = 4; cfg.chunk = 32;
	const int64 b = 1, l = 64;
	// checkpoint-layout (out_features, in_features) float32 weights written as .dat files, then loaded through load_weights
	auto w_in_t = crt_random_normal_tensor<float32, CPU>({ cfg.d_in_proj(), cfg.d_model }, 20, 0.02f);
	auto w_out_t = crt_random_normal_tensor<float32, CPU>({ cfg.d_model, cfg.d_inner }, 21, 0.02f);
	auto conv_w = crt_random_normal_tensor<float32, CPU>({ cfg.conv_dim(), 1, cfg.d_conv }, 22, 0.5f);
	auto conv_b = crt_random_normal_tensor<float32, CPU>({ cfg.conv_dim() }, 23, 0.1f);
	auto norm_w = crt_ones_tensor<float32, CPU>({ cfg.d_inner });
	Tensor<float32, CPU> dt_bias(std::vector<int64>{ cfg.nheads }), A_log(std::vector<int64>{ cfg.nheads }), D(std::vector<int64>{ cfg.nheads });
	for (int64 h = 0; h < cfg.nheads; ++h)
	{
		dt_bias.buffer()[h] = -4.0f + 0.3f * static_cast<float>(h);
		A_log.buffer()[h] = std::log(1.0f + 2.0f * static_cast<float>(h));
		D.buffer()[h] = 1.0f;
	}
	const std::string p = tmp_dir + "/";
	save_tensor(w_in_t, p + "in_proj.dat"); save_tensor(conv_w, p + "conv_w.dat"); save_tensor(conv_b, p + "conv_b.dat");
	save_tensor(dt_bias, p + "dt_bias.dat"); save_tensor(A_log, p + "A_log.dat"); save_tensor(D, p + "D.dat");
	save_tensor(norm_w, p + "norm.dat"); save_tensor(w_out_t, p + "out_proj.dat");
	ZambaMamba2weights<float32> weights;
	weights.load_weights(p + "in_proj.dat", p + "conv_w.dat", p + "conv_b.dat", p + "dt_bias.dat", p + "A_log.dat", p + "D.dat", p + "norm.dat",
		p + "out_proj.dat");
	report("load_weights shapes", weights.in_proj_weight.shape[0] == cfg.d_model && weights.in_proj_weight.shape[1] == cfg.d_in_proj() &&
		weights.conv1d_weight.dim == 2 && weights.out_proj_weight.shape[0] == cfg.d_inner);

	auto u = crt_random_normal_tensor<float32, CPU>({ b, l, cfg.d_model }, 24);
	ZambaMambaCache<float32> cache(cfg, b);
	auto out = tensor_zamba_mamba2_mixer(weights, cache, u.copy_to_cuda(), cfg).copy_to_host();

	auto w_in = weights.in_proj_weight.copy_to_host();    // (in, out) after the load-time transpose
	auto w_out = weights.out_proj_weight.copy_to_host();
	auto cw2 = weights.conv1d_weight.copy_to_host();
	std::vector<float> e(static_cast<size_t>(b * l * cfg.d_model)), efs(static_cast<size_t>(b * cfg.nheads * cfg.headdim * cfg.d_state)),
		ecs(static_cast<size_t>(b * cfg.conv_dim() * (cfg.d_conv - 1)));
	orc_mamba2_mixer_prefill_f32(u.buffer(), w_in.buffer(), cw2.buffer(), conv_b.buffer(), dt_bias.buffer(), A_log.buffer(), D.buffer(),
		norm_w.buffer(), w_out.buffer(), nullptr, e.data(), nullptr, nullptr, nullptr, nullptr, efs.data(), ecs.data(), b, l, cfg.d_model,
		cfg.d_inner, cfg.nheads, cfg.headdim, cfg.ngroups, cfg.d_state, cfg.d_conv, cfg.chunk, cfg.d_inner, cfg.eps, 0);
	report("tensor_zamba_mamba2_mixer f32 prefill", close_enough(out, e, 0.f, 1e-3f));
	report("ZambaMambaCache ssm_state after prefill", close_enough(cache.ssm_state.copy_to_host(), efs, 0.f, 1e-4f));

	// one decode step continues from the cache
	auto u_t = crt_random_normal_tensor<float32, CPU>({ b, cfg.d_model }, 25);
	auto out_t = tensor_zamba_mamba2_mixer(weights, cache, u_t.copy_to_cuda(), cfg).copy_to_host();
	std::vector<float> et(static_cast<size_t>(b * cfg.d_model));
	orc_mamba2_mixer_decode_f32(u_t.buffer(), w_in.buffer(), cw2.buffer(), conv_b.buffer(), dt_bias.buffer(), A_log.buffer(), D.buffer(),
		norm_w.buffer(), w_out.buffer(), ecs.data(), efs.data(), et.data(), b, cfg.d_model, cfg.d_inner, cfg.nheads, cfg.headdim, cfg.ngroups,
		cfg.d_state, cfg.d_conv, cfg.d_inner, cfg.eps, 0);
	report("tensor_zamba_mamba2_mixer f32 decode", close_enough(out_t, et, 0.f, 1e-3f));

	// the same weights from a .safetensors file (F32 and BF16 entries, a __metadata__ object in the header)
	{
		struct Entry { std::string name; const Tensor<float32, CPU>* t; bool bf16; };
		const std::vector<Entry> entries = {
			{ "model.layers.0.mamba.in_proj.weight", &w_in_t, false }, { "model.layers.0.mamba.conv1d.weight", &conv_w, false },
			{ "model.layers.0.mamba.conv1d.bias", &conv_b, false }, { "model.layers.0.mamba.dt_bias", &dt_bias, false },
			{ "model.layers.0.mamba.A_log", &A_log, false }, { "model.layers.0.mamba.D", &D, true },
			{ "model.layers.0.mamba.norm.weight", &norm_w, true }, { "model.layers.0.mamba.out_proj.weight", &w_out_t, false } };
		std::string header = "{\"__metadata__\": {\"format\": \"pt\", \"note\": \"{braces} in a string\"}";
		std::vector<char> data;
		for (const auto& en : entries)
		{
			const size_t n = static_cast<size_t>(en.t->numel());
			const size_t begin = data.size();
			if (en.bf16)  // D and the norm weight are all ones: exact in bfloat16
				for (size_t i = 0; i < n; ++i)
				{
					uint32_t u;
					std::memcpy(&u, &en.t->buffer()[i], 4);
					const uint16_t b16 = static_cast<uint16_t>(u >> 16);
					data.insert(data.end(), reinterpret_cast<const char*>(&b16), reinterpret_cast<const char*>(&b16) + 2);
				}
			else
				data.insert(data.end(), reinterpret_cast<const char*>(en.t->buffer()), reinterpret_cast<const char*>(en.t->buffer()) + n * 4);
			header += ", \"" + en.name + "\": {\"dtype\": \"" + (en.bf16 ? "BF16" : "F32") + "\", \"shape\": [";
			for (int64 k = 0; k < en.t->dim; ++k) header += (k ? ", " : "") + std::to_string(en.t->shape[k]);
			header += "], \"data_offsets\": [" + std::to_string(begin) + ", " + std::to_string(data.size()) + "]}";
		}
		header += "}";
		while (header.size() % 8) header.push_back(' ');
		{
			std::ofstream f(p + "mixer.safetensors", std::ios::binary);
			const unsigned long long hs = header.size();
			f.write(reinterpret_cast<const char*>(&hs), 8);
			f.write(header.data(), static_cast<std::streamsize>(header.size()));
			f.write(data.data(), static_cast<std::streamsize>(data.size()));
		}
		const auto infos = sft_read_tensorinfos(p + "mixer.safetensors");
		report("safetensors header: 8 tensors, metadata skipped", infos.size() == 8 && infos[1].shape.size() == 3 && infos[5].dtype == "BF16");
		ZambaMamba2weights<float32> sw;
		sw.load_safetensors(p + "mixer.safetensors", "model.layers.0.mamba.");
		auto same = [](const auto& a, const auto& b) {
			auto ha = a.copy_to_host(), hb = b.copy_to_host();
			return ha.numel() == hb.numel() && std::memcmp(ha.buffer(), hb.buffer(), sizeof(*ha.buffer()) * static_cast<size_t>(ha.numel())) == 0;
		};
		report("load_safetensors equals load_weights", same(sw.in_proj_weight, weights.in_proj_weight) && same(sw.conv1d_weight, weights.conv1d_weight) &&
			same(sw.conv1d_bias, weights.conv1d_bias) && same(sw.dt_bias, weights.dt_bias) && same(sw.A_log, weights.A_log) && same(sw.D, weights.D) &&
			same(sw.norm_weight, weights.norm_weight) && same(sw.out_proj_weight, weights.out_proj_weight));
	}

	// the same prompt in two pieces (40 + 24 tokens; 40 is not a multiple of the chunk) from a fresh cache
	{
		ZambaMambaCache<float32> pc(cfg, b);
		// batch 1: a token range of u is a contiguous block
		auto piece = [&](int64 t0, int64 t1) {
			std::vector<float32> h(u.buffer() + t0 * cfg.d_model, u.buffer() + t1 * cfg.d_model);
			return Tensor<float32, CPU>(std::vector<int64>{ b, t1 - t0, cfg.d_model }, h).copy_to_cuda();
		};
		auto o1 = tensor_zamba_mamba2_mixer_continue(weights, pc, piece(0, 40), cfg).copy_to_host();
		auto o2 = tensor_zamba_mamba2_mixer_continue(weights, pc, piece(40, l), cfg).copy_to_host();
		const std::vector<float> e1(e.begin(), e.begin() + 40 * cfg.d_model), e2(e.begin() + 40 * cfg.d_model, e.end());
		report("tensor_zamba_mamba2_mixer_continue f32, first piece of the prompt", close_enough(o1, e1, 0.f, 1e-3f));
		report("tensor_zamba_mamba2_mixer_continue f32, second piece of the prompt", close_enough(o2, e2, 0.f, 1e-3f));

		// a packed batch of two sequences: the prompt and its first 40 tokens (causal: the same first 40 outputs)
		std::vector<float32> packed(u.buffer(), u.buffer() + l * cfg.d_model);
		packed.insert(packed.end(), u.buffer(), u.buffer() + 40 * cfg.d_model);
		ZambaMambaCache<float32> vc(cfg, 2);
		auto vo = tensor_zamba_mamba2_mixer_varlen(weights, vc, Tensor<float32, CPU>(std::vector<int64>{ l + 40, cfg.d_model }, packed).copy_to_cuda(),
			std::vector<int64>{ 0, l, l + 40 }, cfg).copy_to_host();
		const Tensor<float32, CPU> v1(std::vector<int64>{ l, cfg.d_model }, std::vector<float32>(vo.buffer(), vo.buffer() + l * cfg.d_model));
		const Tensor<float32, CPU> v2(std::vector<int64>{ 40, cfg.d_model },
			std::vector<float32>(vo.buffer() + l * cfg.d_model, vo.buffer() + (l + 40) * cfg.d_model));
		report("tensor_zamba_mamba2_mixer_varlen f32, first sequence", close_enough(v1, e, 0.f, 1e-3f));
		report("tensor_zamba_mamba2_mixer_varlen f32, second sequence", close_enough(v2, e1, 0.f, 1e-3f));
	}

	// the decoder layer around the same mixer: y = h + mixer(rms_norm(h) * w_in), prefill then one decode step
	auto in_norm = crt_random_normal_tensor<float32, CPU>({ cfg.d_model }, 26, 0.1f);
	for (int64 i = 0; i < cfg.d_model; ++i) in_norm.buffer()[i] += 1.0f;
	save_tensor(in_norm, p + "in_norm.dat");
	ZambaMambaDecoderweights<float32> dw;
	dw.load_weights(p + "in_norm.dat", p + "in_proj.dat", p + "conv_w.dat", p + "conv_b.dat", p + "dt_bias.dat", p + "A_log.dat", p + "D.dat",
		p + "norm.dat", p + "out_proj.dat");
	ZambaMambaCache<float32> dcache(cfg, b);
	auto dout = tensor_zamba_mamba_decoder(dw, dcache, u.copy_to_cuda(), cfg, 1e-5f).copy_to_host();
	std::vector<float> normed(static_cast<size_t>(b * l * cfg.d_model)), de(normed.size());
	orc_rms_norm_f32(u.buffer(), in_norm.buffer(), normed.data(), b * l, cfg.d_model, 1e-5f, 0);
	orc_mamba2_mixer_prefill_f32(normed.data(), w_in.buffer(), cw2.buffer(), conv_b.buffer(), dt_bias.buffer(), A_log.buffer(), D.buffer(),
		norm_w.buffer(), w_out.buffer(), nullptr, de.data(), nullptr, nullptr, nullptr, nullptr, efs.data(), ecs.data(), b, l, cfg.d_model,
		cfg.d_inner, cfg.nheads, cfg.headdim, cfg.ngroups, cfg.d_state, cfg.d_conv, cfg.chunk, cfg.d_inner, cfg.eps, 0);
	for (size_t i = 0; i < de.size(); ++i) de[i] += u.buffer()[i];
	report("tensor_zamba_mamba_decoder f32 prefill", close_enough(dout, de, 0.f, 1e-3f));
	auto dout_t = tensor_zamba_mamba_decoder(dw, dcache, u_t.copy_to_cuda(), cfg, 1e-5f).copy_to_host();
	std::vector<float> normed_t(static_cast<size_t>(b * cfg.d_model));
	orc_rms_norm_f32(u_t.buffer(), in_norm.buffer(), normed_t.data(), b, cfg.d_model, 1e-5f, 0);
	orc_mamba2_mixer_decode_f32(normed_t.data(), w_in.buffer(), cw2.buffer(), conv_b.buffer(), dt_bias.buffer(), A_log.buffer(), D.buffer(),
		norm_w.buffer(), w_out.buffer(), ecs.data(), efs.data(), et.data(), b, cfg.d_model, cfg.d_inner, cfg.nheads, cfg.headdim, cfg.ngroups,
		cfg.d_state, cfg.d_conv, cfg.d_inner, cfg.eps, 0);
	for (size_t i = 0; i < et.size(); ++i) et[i] += u_t.buffer()[i];
	report("tensor_zamba_mamba_decoder f32 decode", close_enough(dout_t, et, 0.f, 1e-3f));
}

// tensor_slice under anyGPU's name (srcs/ops/shape_ops.hpp:190-254): a contiguous copy of x[..., lo:hi, ...] along any axis, on both
// devices; and the zero fill of a fresh device tensor that anyGPU's MemoryBuffer guarantees (srcs/core/tensor.hpp:80-84).
static void test_tensor_slice_and_zero_fill()
{
	const int64 b = 3, l = 5, d = 14;
	auto h = crt_random_normal_tensor<float32, CPU>({ b, l, d }, 7);
	auto dv = h.copy_to_cuda();
	bool ok = true;
	const int64 cases[3][3] = { { 2, 4, 11 }, { 1, 1, 4 }, { 0, 2, 3 } };
	for (const auto& c : cases)
	{
		const int64 axis = c[0], lo = c[1], hi = c[2];
		auto g = tensor_slice(dv, axis, lo, hi).copy_to_host();
		auto e = tensor_slice(h, axis, lo, hi);
		Shape want = h.shape;
		want[axis] = hi - lo;
		ok = ok && g.dim == 3 && g.shape == want && e.shape == want;
		for (int64 i = 0; i < want[0] && ok; ++i)
			for (int64 j = 0; j < want[1]; ++j)
				for (int64 k = 0; k < want[2]; ++k)
				{
					const int64 si = i + (axis == 0 ? lo : 0), sj = j + (axis == 1 ? lo : 0), sk = k + (axis == 2 ? lo : 0);
					const float ref = h.buffer()[(si * l + sj) * d + sk];
					const int64 o = (i * want[1] + j) * want[2] + k;
					ok = ok && g.buffer()[o] == ref && e.buffer()[o] == ref;
				}
	}
	report("tensor_slice (axes 0, 1, 2; CPU and CUDA)", ok);
	Tensor<float32, CUDA> fresh({ 7, 33 });
	auto fh = fresh.copy_to_host();
	bool zero = true;
	for (int64 i = 0; i < fh.numel(); ++i) zero = zero && fh.buffer()[i] == 0.f;
	report("fresh device tensor is zero-filled", zero);
}

int main(int argc, char** argv)
{
	const std::string tmp_dir = argc > 1 ? argv[1] : "/tmp";
	int ndev = 0;
	if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0)
	{
		std::printf("no CUDA device: this library has no CPU path\n");
		return 2;
	}
	test_causal_conv1d_f16();
	test_linear_f16();
	test_gated_rmsnorm_f32();
	test_rms_norm();
	test_chunk_scan_f16();
	test_mixer_f32_and_dat_files(tmp_dir);
	test_tensor_slice_and_zero_fill();
	CUDA_CHECK(cudaDeviceSynchronize());
	uint32_t detail = 0;
	report("no device-side timeout", b200_last_device_error(nullptr, &detail) == B200_OK);
	std::printf("Finished: %d failed\n", g_failed);
	return g_failed == 0 ? 0 : 1;
}
