// SSD chunked scan for callers that cannot hand over scratch memory.
//
// b200_mamba_chunk_scan_combined needs a caller-provided workspace. Some hosts have nowhere to get one from: a plugin
// that is only handed its input and output tensors by a runtime which owns the device allocator, code running inside a
// region where cudaMalloc is forbidden (a stream capture, a real-time loop with a no-allocation rule), or a binding
// whose memory pool cannot grow any more. For them this file keeps a fixed scratch array inside the library's own
// device image and runs the same four stages on it.
//
// The array costs kStaticScratchBytes of device memory on EVERY GPU that loads the library, from module load until the
// process exits, whether or not this entry point is ever called.
#include <mutex>

#include "ssd_common.cuh"

namespace b200 {

constexpr size_t kStaticScratchBytes = 64ull << 20;  // 64 MiB: enough for batch 4 x 2048 tokens, 64 heads x 64 x 64, chunk 256

// In host code this name is only a handle for the runtime's symbol table, not a device address: launching a kernel with
// `g_static_scratch` itself as an argument would pass a HOST address. The device address is obtained below with
// cudaGetSymbolAddress, once per device.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

static int static_scratch_address(void** out)
{
	static std::mutex mu;
	static void* addr[64] = {};
	int dev = -1;
	B200_CUDA_TRY(cudaGetDevice(&dev));
	if (dev < 0 || dev >= 64) return B200_ERR_UNSUPPORTED;
	std::lock_guard<std::mutex> lk(mu);
	if (!addr[dev])
	{
		// the current device is `dev`: the address returned is that device's copy of the array
		void* p = nullptr;
		B200_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_scratch));
		addr[dev] = p;
	}
	*out = addr[dev];
	return B200_OK;
}

}  // namespace b200

using namespace b200;

extern "C" size_t b200_mamba_chunk_scan_combined_static_capacity(void) { return kStaticScratchBytes; }

extern "C" int b200_mamba_chunk_scan_combined_static(int dtype, const void* x, int64_t x_stride, const void* dt, int64_t dt_stride,
	const float* A, int a_is_log, const void* B, int64_t B_stride, const void* C, int64_t C_stride,
	const float* D, const float* dt_bias, const float* initial_states,
	void* y, int64_t y_stride, float* final_states,
	int64_t batch, int64_t seqlen, int64_t H, int64_t P, int64_t G, int64_t N, int64_t chunk, int dt_softplus, void* stream)
{
	if (batch < 0 || seqlen < 0 || H <= 0 || P <= 0 || G <= 0 || N <= 0 || chunk <= 0) return B200_ERR_BAD_SHAPE;
	if (batch == 0 || seqlen == 0) return B200_OK;
	const size_t need = b200_mamba_chunk_scan_combined_workspace_bytes(batch, seqlen, H, P, G, N, chunk);
	if (need == 0) return B200_ERR_BAD_SHAPE;
	if (need > kStaticScratchBytes) return B200_ERR_WORKSPACE;  // problem too large for the built-in scratch
	void* scratch = nullptr;
	const int rc = static_scratch_address(&scratch);
	if (rc) return rc;
	// Every word of the scratch that a stage reads was written earlier in the same call (dt and dAcs by stage 1,
	// the chunk states by stage 2, the passed states by stage 3), so nothing has to be cleared between calls.
	return b200_mamba_chunk_scan_combined(dtype, x, x_stride, dt, dt_stride, A, a_is_log, B, B_stride, C, C_stride, D, dt_bias,
		initial_states, y, y_stride, final_states, batch, seqlen, H, P, G, N, chunk, dt_softplus, scratch, kStaticScratchBytes, stream);
}
