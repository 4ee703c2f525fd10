// Library-wide state of the C ABI: status strings, the per-thread CUDA error record and the device error word
// that bounded device-side waits set when they give up.
#include "common.cuh"
#include <atomic>
#include <cstdlib>

namespace b200 {

thread_local int g_last_cuda_error = 0;

static std::atomic<long long> g_launches{ 0 };
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

__device__ uint32_t g_device_error_word = 0;

bool pdl_enabled()
{
	static const bool on = [] {
		const char* v = getenv("B200_NO_PDL");
		return !(v && v[0] == '1');
	}();
	return on;
}

uint32_t* device_error_word()
{
	// one address per device; a process drives one GPU in this design, but stay correct if it drives several
	static uint32_t* addr[64] = {};
	int dev = 0;
	if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
	if (!addr[dev])
	{
		void* p = nullptr;
		if (cudaGetSymbolAddress(&p, g_device_error_word) != cudaSuccess) return nullptr;
		addr[dev] = static_cast<uint32_t*>(p);
	}
	return addr[dev];
}

}  // namespace b200

using namespace b200;

extern "C" const char* b200_status_string(int status)
{
	switch (status)
	{
	case B200_OK: return "ok";
	case B200_ERR_BAD_SHAPE: return "bad shape";
	case B200_ERR_MISALIGNED: return "misaligned pointer or stride";
	case B200_ERR_WORKSPACE: return "workspace missing or too small";
	case B200_ERR_DEVICE_TIMEOUT: return "device-side wait timed out";
	case B200_ERR_CUDA: return "CUDA call failed";
	case B200_ERR_UNSUPPORTED: return "unsupported dtype or size";
	case B200_ERR_NULL: return "null pointer";
	default: return "unknown status";
	}
}

extern "C" int b200_last_cuda_error(void) { return g_last_cuda_error; }

extern "C" int b200_abi_version(void) { return 3; }

extern "C" long long b200_launch_count(int reset)
{
	return reset ? g_launches.exchange(0, std::memory_order_relaxed) : g_launches.load(std::memory_order_relaxed);
}

extern "C" int b200_last_device_error(void* stream, uint32_t* detail)
{
	uint32_t* word = device_error_word();
	if (!word) return B200_ERR_CUDA;
	cudaStream_t st = static_cast<cudaStream_t>(stream);
	uint32_t v = 0;
	B200_CUDA_TRY(cudaMemcpyAsync(&v, word, sizeof(v), cudaMemcpyDeviceToHost, st));
	B200_CUDA_TRY(cudaStreamSynchronize(st));
	if (detail) *detail = v;
	if (v != 0)
	{
		B200_CUDA_TRY(cudaMemsetAsync(word, 0, sizeof(v), st));
		B200_CUDA_TRY(cudaStreamSynchronize(st));
		return B200_ERR_DEVICE_TIMEOUT;
	}
	return B200_OK;
}
