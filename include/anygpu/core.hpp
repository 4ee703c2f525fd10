// Core definitions of the header layer: the names a caller of anyGPU's operators relies on (dtype aliases, Shape /
// Stride arrays, Device, logging, ACASSERT, CUDA_CHECK), written for this library. Interface reference:
// anyGPU srcs/core/core.hpp:32-41 (dtype aliases), :60-66 (DimArray), :74-78 (Device), :365-422 (log_*, ACASSERT),
// :445-475 (CUDA_CHECK*). Header-only; needs the CUDA runtime headers and cuda_fp16.h.
#pragma once

#include <array>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <iostream>
#include <sstream>
#include <string>
#include <vector>

#include <cuda_fp16.h>
#include <cuda_runtime.h>

using int8 = char;
using int16 = short signed int;
using int32 = signed int;
using int64 = long long;
using float16 = half;
using float32 = float;
using float64 = double;

constexpr int MAX_TENSOR_DIM = 8;
using DimArray = std::array<int64, MAX_TENSOR_DIM>;
using Shape = DimArray;
using Stride = DimArray;

enum Device
{
	CPU,
	CUDA
};

inline void log_info(const std::string& msg) { std::cout << "[info] " << msg << std::endl; }
inline void log_warning(const std::string& msg) { std::cout << "[warning] " << msg << std::endl; }
inline void log_error(const std::string& msg) { std::cout << "[error] " << msg << std::endl; }

// Same contract as anyGPU's ACASSERT: print location + message and exit(1); compiled out without AC_WITH_ASSERT.
#ifdef AC_WITH_ASSERT
#define ACASSERT(expression, msg)                              \
	do {                                                       \
		if (!(expression))                                     \
		{                                                      \
			std::cout << __FILE__ << " " << __LINE__ << '\n';  \
			log_error(msg);                                    \
			exit(1);                                           \
		}                                                      \
	} while (0)
#else
#define ACASSERT(expression, msg) ((void)0)
#endif

#define CUDA_CHECK(fn)                                                                     \
	do {                                                                                   \
		cudaError_t res__ = (fn);                                                          \
		if (res__ != cudaSuccess)                                                          \
		{                                                                                  \
			std::stringstream ss__;                                                        \
			ss__ << "code: " << (int)res__ << " file: " << __FILE__ << " ln: " << __LINE__; \
			log_error(ss__.str());                                                         \
			exit(1);                                                                       \
		}                                                                                  \
	} while (0)

#define CUDA_CHECK_LAST_ERROR() CUDA_CHECK(cudaGetLastError())

inline int64 calc_default_size(const std::vector<int64>& shape)
{
	int64 n = 1;
	for (int64 s : shape) n *= s;
	return n;
}

inline int64 calc_default_size(const int64 dim, const DimArray& shape)
{
	int64 n = 1;
	for (int64 i = 0; i < dim; ++i) n *= shape[i];
	return n;
}

inline DimArray calc_default_stride(const int64 dim, const DimArray& shape)
{
	DimArray st{};
	int64 acc = 1;
	for (int64 i = dim - 1; i >= 0; --i)
	{
		st[i] = acc;
		acc *= shape[i];
	}
	return st;
}

inline DimArray cvt_vector2array(const std::vector<int64>& v)
{
	DimArray a{};
	for (size_t i = 0; i < v.size() && i < static_cast<size_t>(MAX_TENSOR_DIM); ++i) a[i] = v[i];
	return a;
}

class GlobalUUIDGenerator
{
public:
	static int64 generate_id()
	{
		static int64 next_id = 0;
		return next_id++;
	}
};
