// Timing program around the reference's OWN CUDA kernels, compiled for sm_100a from the reference sources where they lie
// (nothing is copied: the Makefile passes the reference's .cu files to nvcc beside this one). It is the "reference kernels
// recompiled for this GPU" baseline that bench.py reports next to this repository's kernels.
//
// TEST / MEASUREMENT INFRASTRUCTURE ONLY: the shipped library never loads it. It runs as a process of its own, because the
// reference's launchers call exit(1) on any CUDA error (srcs/core/core.hpp:461-475).
//
// Kernels timed (shapes chosen after reading the kernels' index arithmetic):
//   opt2::cu_tensor_mm_f16   srcs/kernels/cuda/mm_ops.cu:231-350  f16 SIMT tile kernel, f16 accumulation, no bounds checks:
//                            M, N, K must be multiples of 64 -> the cfg2 projections (8192x2048x8384, 8192x4096x2048) qualify
//   cu_tensor_causal_conv1d_f32  srcs/kernels/cuda/causal_conv1d.cu:7-101  f32 only; (8, 4224, 4096) as in the conv configuration
// Not run: cu_tensor_rms_norm_f32_v1 (norm_rms_f32_v1.cu:94-119) copies the weight into a 1344-float __constant__ array
// whatever its length, so it cannot take the 4096-wide rows of this path.
//
// usage: ref_cuda_bench <mm|conv> <steps>   -> one JSON line
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "tensor.hpp"
#include "mm_ops.cuh"
#include "causal_conv1d.cuh"

static Tensor<float16, CUDA> random_f16(const std::vector<int64>& shape, int64 seed, float scale)
{
	auto f = crt_random_normal_tensor<float32, CPU>(shape, seed);
	Tensor<float16, CPU> h(shape);
	for (int64 i = 0; i < h.size(); ++i) h.buffer()[i] = __float2half(f.buffer()[i] * scale);
	return h.copy_to_cuda();
}

template <typename F>
static float time_ms(int steps, F&& fn)
{
	cudaEvent_t e0, e1;
	cudaEventCreate(&e0);
	cudaEventCreate(&e1);
	fn();  // warm-up
	cudaDeviceSynchronize();
	cudaEventRecord(e0);
	for (int i = 0; i < steps; ++i) fn();
	cudaEventRecord(e1);
	cudaEventSynchronize(e1);
	float ms = 0.f;
	cudaEventElapsedTime(&ms, e0, e1);
	return ms / static_cast<float>(steps);
}

int main(int argc, char** argv)
{
	if (argc < 3) return 2;
	const std::string what = argv[1];
	const int steps = std::atoi(argv[2]);
	int ndev = 0;
	if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0)
	{
		std::printf("{\"unavailable\": \"no CUDA device\"}\n");
		return 0;
	}
	if (what == "mm")
	{
		struct Shape3 { long long m, k, n; const char* name; };
		const Shape3 shapes[2] = { { 8192, 2048, 8384, "in_proj" }, { 8192, 4096, 2048, "out_proj" } };
		std::printf("{\"kernel\": \"opt2::cu_tensor_mm_f16\"");
		for (const auto& s : shapes)
		{
			auto lhs = random_f16({ s.m, s.k }, 1, 1.0f);
			auto rhs = random_f16({ s.k, s.n }, 2, 0.02f);
			Tensor<float16, CUDA> out(std::vector<int64>{ s.m, s.n });
			const float ms = time_ms(steps, [&] { opt2::cu_tensor_mm_f16(lhs, rhs, out); });
			std::printf(", \"%s_ms\": %.4f, \"%s_tflops\": %.3f", s.name, ms, s.name, 2.0 * s.m * s.k * s.n / (ms * 1e-3) / 1e12);
		}
		std::printf("}\n");
	}
	else if (what == "conv")
	{
		const long long b = 8, d = 4224, l = 4096, w = 4;
		auto x = crt_random_normal_tensor<float32, CPU>({ b, d, l }, 3).copy_to_cuda();
		auto wt = crt_random_normal_tensor<float32, CPU>({ d, w }, 4).copy_to_cuda();
		auto bt = crt_random_normal_tensor<float32, CPU>({ d }, 5).copy_to_cuda();
		Tensor<float32, CUDA> y(std::vector<int64>{ b, d, l });
		const float ms = time_ms(steps, [&] { cu_tensor_causal_conv1d_f32(x, wt, bt, y); });
		std::printf("{\"kernel\": \"cu_tensor_causal_conv1d_f32\", \"shape\": [%lld, %lld, %lld], \"ms\": %.4f, \"gbs\": %.1f}\n", b, d, l, ms,
			2.0 * b * d * l * 4 / (ms * 1e-3) / 1e9);
	}
	else
		return 2;
	return 0;
}
