// Reader / writer of anyGPU's .dat tensor files (format described in srcs/io/dat_file.hpp:6-27 and written by
// scripts/dnn_inspector/dnninspect/tensor.py:76-142): int32 dim, int32 shape[dim], int32 dtype code
// (2 int32, 4 float16, 5 float32, 6 float64), then the raw elements with default strides.
#pragma once

#include <fstream>

#include "../tensor.hpp"

template <typename T>
constexpr int dat_dtype_code()
{
	if constexpr (std::is_same_v<T, int32>) return 2;
	else if constexpr (std::is_same_v<T, float16>) return 4;
	else if constexpr (std::is_same_v<T, float32>) return 5;
	else
	{
		static_assert(std::is_same_v<T, float64>, "unsupported .dat element type");
		return 6;
	}
}

template <typename T = float32>
inline Tensor<T, CPU> load_tensor(const std::string& file_path)
{
	std::ifstream f(file_path, std::ios::binary);
	if (!f.is_open())
	{
		log_error("Unable to open file: " + file_path);
		exit(1);
	}
	int32 dim = 0;
	f.read(reinterpret_cast<char*>(&dim), sizeof(int32));
	std::vector<int64> shape(static_cast<size_t>(dim));
	for (auto& s : shape)
	{
		int32 v = 0;
		f.read(reinterpret_cast<char*>(&v), sizeof(int32));
		s = v;
	}
	int32 code = 0;
	f.read(reinterpret_cast<char*>(&code), sizeof(int32));
	if (code != dat_dtype_code<T>())
	{
		log_error("Data type in tensor data file does not match the requested element type: " + file_path);
		exit(1);
	}
	Tensor<T, CPU> t(shape);
	f.read(reinterpret_cast<char*>(t.buffer()), static_cast<std::streamsize>(sizeof(T) * t.numel()));
	return t;
}

template <typename T>
inline void save_tensor(const Tensor<T, CPU>& t, const std::string& file_path)
{
	std::ofstream f(file_path, std::ios::binary);
	const int32 dim = static_cast<int32>(t.dim);
	f.write(reinterpret_cast<const char*>(&dim), sizeof(int32));
	for (int64 i = 0; i < t.dim; ++i)
	{
		const int32 v = static_cast<int32>(t.shape[i]);
		f.write(reinterpret_cast<const char*>(&v), sizeof(int32));
	}
	const int32 code = dat_dtype_code<T>();
	f.write(reinterpret_cast<const char*>(&code), sizeof(int32));
	f.write(reinterpret_cast<const char*>(t.buffer()), static_cast<std::streamsize>(sizeof(T) * t.numel()));
}
