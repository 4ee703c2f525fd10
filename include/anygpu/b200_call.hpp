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

// Returns a device buffer of at least `bytes` bytes that stays valid until the next larger request on this thread.
inline void* b200_workspace(const size_t bytes)
{
	thread_local std::shared_ptr<MemoryBuffer<CUDA>> ws;
	if (!ws || static_cast<size_t>(ws->capacity) < bytes)
	{
		CUDA_CHECK(cudaDeviceSynchronize());  // kernels may still be using the old buffer
		ws = std::make_shared<MemoryBuffer<CUDA>>(static_cast<int64>(bytes < 256 ? 256 : bytes));
	}
	return ws->buffer;
}
