// Glue between the tensor_<op> templates and the C ABI: dtype tag, status handling in anyGPU's style
// (log_error + exit(1), srcs/core/core.hpp:408-475), and a grow-only device workspace owned by the caller's thread
// (the "arena" that anyGPU's own TODO asks for, docs/TODO.md:42-47) so that operators do not allocate per call.
#pragma once

#include <type_traits>

#include "b200_mamba2.h"
#include "tensor.hpp"

template <typename dtype>
constexpr int b200_dtype_of()
{
	static_assert(std::is_same_v<dtype, float16> || std::is_same_v<dtype, float32>, "Unsupported data types");
	return std::is_same_v<dtype, float16> ? B200_F16 : B200_F32;
}

inline void b200_check(const int status, const char* what)
{
	if (status == B200_OK) return;
	std::stringstream ss;
	ss << what << ": " << b200_status_string(status) << " (status " << status << ", cuda error " << b200_last_cuda_error() << ")";
	log_error(ss.str());
	exit(1);
}

// Returns a buffer of at least `bytes` bytes on the CURRENT device that stays valid until the next larger request of this
// thread on that device (one buffer per thread and device: after cudaSetDevice the other device's buffer is not handed out).
inline void* b200_workspace(const size_t bytes)
{
	constexpr int kMaxDevices = 64;
	thread_local std::shared_ptr<MemoryBuffer<CUDA>> ws[kMaxDevices];
	int dev = 0;
	CUDA_CHECK(cudaGetDevice(&dev));
	if (dev < 0 || dev >= kMaxDevices)
	{
		log_error("b200_workspace: device index out of range");
		exit(1);
	}
	if (!ws[dev] || static_cast<size_t>(ws[dev]->capacity) < bytes)
	{
		CUDA_CHECK(cudaDeviceSynchronize());  // kernels may still be using the old buffer
		ws[dev] = std::make_shared<MemoryBuffer<CUDA>>(static_cast<int64>(bytes < 256 ? 256 : bytes));
	}
	return ws[dev]->buffer;
}
