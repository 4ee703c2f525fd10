// Shared device/host helpers for the B200 Mamba2-mixer kernels (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stddef.h>

#include "b200_mamba2.h"

#if defined(__CUDA_ARCH__) && (__CUDA_ARCH__ < 1000)
#error "these kernels are written for sm_100a only"
#endif

namespace b200 {

// ---- host side -------------------------------------------------------------------------------------------

extern thread_local int g_last_cuda_error;

inline int record_cuda(cudaError_t e)
{
	if (e == cudaSuccess) return B200_OK;
	g_last_cuda_error = static_cast<int>(e);
	return B200_ERR_CUDA;
}

#define B200_CUDA_TRY(expr)                                   \
	do {                                                      \
		cudaError_t e__ = (expr);                             \
		if (e__ != cudaSuccess) return b200::record_cuda(e__); \
	} while (0)

// Kernel launches issued by the library in this process (b200_launch_count reads and resets it): every launch site passes
// through B200_LAUNCH_CHECK or launch_chained.
void count_launch();

// Launch check that does not synchronise.
#define B200_LAUNCH_CHECK()                \
	do {                                   \
		b200::count_launch();              \
		B200_CUDA_TRY(cudaGetLastError()); \
	} while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline int64_t cdiv(int64_t a, int64_t b) { return (a + b - 1) / b; }
inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

constexpr int kNumSMs = 148;  // B200: 2 dies x 74 SMs

// Device-side error word set by bounded waits (0 = none).
uint32_t* device_error_word();

// Kernel launch with programmatic stream serialization (see pdl_wait below); `pdl` false gives a normal launch.
// Opt-in to more than 48 KiB of dynamic shared memory, once per device and kernel (the attribute belongs to the device's
// context: a process that drives several GPUs needs it on each). `done` is the call site's static per-device flag array.
template <typename K>
inline cudaError_t allow_dynamic_smem(K* kernel, int bytes, bool (&done)[64])
{
	int dev = 0;
	cudaError_t e = cudaGetDevice(&dev);
	if (e != cudaSuccess) return e;
	if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
	if (done[dev]) return cudaSuccess;
	e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
	if (e == cudaSuccess) done[dev] = true;
	return e;
}

bool pdl_enabled();  // false when the environment variable B200_NO_PDL is set to 1
template <typename... KArgs, typename... Args>
inline cudaError_t launch_chained(bool pdl, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args)
{
	cudaLaunchConfig_t cfg = {};
	cfg.gridDim = grid;
	cfg.blockDim = block;
	cfg.dynamicSmemBytes = smem;
	cfg.stream = st;
	cudaLaunchAttribute attr[1];
	attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
	attr[0].val.programmaticStreamSerializationAllowed = 1;
	cfg.attrs = attr;
	cfg.numAttrs = pdl ? 1 : 0;
	count_launch();
	return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ---- device side -----------------------------------------------------------------------------------------

template <typename T> struct Cvt;
template <> struct Cvt<float>
{
	static __device__ __forceinline__ float to_f32(float v) { return v; }
	static __device__ __forceinline__ float from_f32(float v) { return v; }
};
template <> struct Cvt<__half>
{
	static __device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
	static __device__ __forceinline__ __half from_f32(float v) { return __float2half_rn(v); }
};

template <typename T> __device__ __forceinline__ float ldf(const T* p) { return Cvt<T>::to_f32(*p); }
template <typename T> __device__ __forceinline__ void stf(T* p, float v) { *p = Cvt<T>::from_f32(v); }

// silu(x) = x / (1 + exp(-x)), the form anyGPU uses (srcs/kernels/cuda/math_ops.cu:3-34).
// The quotient uses the fast reciprocal path (2 ulp): an IEEE division here makes the conv and norm kernels
// instruction-bound instead of HBM-bound.
__device__ __forceinline__ float silu_f32(float v)
{
	// ex2 / rcp in their flush-to-zero forms: the default forms wrap each MUFU in range checks and rescaling for denormals,
	// which nothing here can tell apart from zero (v < -87 gives -0 instead of a denormal)
	float e, r;
	asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(v * -1.4426950408889634f));
	asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
	return v * r;
}

// torch softplus (beta 1, threshold 20), as F.softplus in scripts/zamba2/mamba_chunk_scan_comb.py:45.
__device__ __forceinline__ float softplus_f32(float v) { return v > 20.f ? v : log1pf(expf(v)); }

// Programmatic dependent launch: a kernel launched with programmatic stream serialization may start while the kernel before
// it in the stream still runs. pdl_wait() blocks until that kernel has completed and its writes are visible (a no-op for a
// normal launch); pdl_launch_dependents() lets the kernel after this one start once every CTA here has issued it or exited.
// Rules kept by every kernel of such a chain: only constant data (weights) is touched before pdl_wait(), and every CTA
// executes pdl_wait() before it exits, so that completion of a kernel implies completion of everything before it.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
	for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
	return v;
}

// 8 f16 values <-> 8 floats through one 128-bit access
struct alignas(16) Half8
{
	__half2 h[4];
};

__device__ __forceinline__ void unpack8(const Half8& v, float* f)
{
#pragma unroll
	for (int i = 0; i < 4; ++i)
	{
		float2 t = __half22float2(v.h[i]);
		f[2 * i] = t.x;
		f[2 * i + 1] = t.y;
	}
}

__device__ __forceinline__ Half8 pack8(const float* f)
{
	Half8 v;
#pragma unroll
	for (int i = 0; i < 4; ++i) v.h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
	return v;
}

// V consecutive elements of T moved with one access of V*sizeof(T) bytes (16, 8, 4 or 2).
template <int BYTES> struct BitsOf;
template <> struct BitsOf<16> { using type = uint4; };
template <> struct BitsOf<8> { using type = uint2; };
template <> struct BitsOf<4> { using type = uint32_t; };
template <> struct BitsOf<2> { using type = uint16_t; };

template <typename T, int V>
struct Pack
{
	using B = typename BitsOf<V * sizeof(T)>::type;
	B bits;
	__device__ __forceinline__ void load(const T* p) { bits = *reinterpret_cast<const B*>(p); }
	// 8- or 16-byte load that stays where it is written (the compiler may otherwise move a load down to its first use and
	// serialise what was meant to be a batch of independent requests)
	__device__ __forceinline__ void load_pinned(const T* p)
	{
		static_assert(V * sizeof(T) == 16 || V * sizeof(T) == 8, "load_pinned moves 8 or 16 bytes");
		if constexpr (V * sizeof(T) == 16)
			asm volatile("ld.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(bits.x), "=r"(bits.y), "=r"(bits.z), "=r"(bits.w) : "l"(p) : "memory");
		else
			asm volatile("ld.global.v2.u32 {%0, %1}, [%2];" : "=r"(bits.x), "=r"(bits.y) : "l"(p) : "memory");
	}
	// The same for data that is read once: the lines are marked first to leave L2, so that what the kernel writes (the next
	// kernel's input) is what stays there.
	__device__ __forceinline__ void load_pinned_once(const T* p)
	{
		static_assert(V * sizeof(T) == 16, "load_pinned_once moves 16 bytes");
		uint64_t pol;
		asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
		asm volatile("ld.global.L2::cache_hint.v4.u32 {%0, %1, %2, %3}, [%4], %5;"
			: "=r"(bits.x), "=r"(bits.y), "=r"(bits.z), "=r"(bits.w) : "l"(p), "l"(pol) : "memory");
	}
	__device__ __forceinline__ void store(T* p) const { *reinterpret_cast<B*>(p) = bits; }
	// f16 pairs go through the packed half2 conversions (a scalar f16 -> f32 conversion issues on the slow XU pipe)
	__device__ __forceinline__ void unpack(float* f) const
	{
		if constexpr (sizeof(T) == 2 && V % 2 == 0)
		{
			const __half2* e = reinterpret_cast<const __half2*>(&bits);
#pragma unroll
			for (int i = 0; i < V / 2; ++i)
			{
				const float2 t = __half22float2(e[i]);
				f[2 * i] = t.x;
				f[2 * i + 1] = t.y;
			}
		}
		else
		{
			const T* e = reinterpret_cast<const T*>(&bits);
#pragma unroll
			for (int i = 0; i < V; ++i) f[i] = Cvt<T>::to_f32(e[i]);
		}
	}
	__device__ __forceinline__ void pack(const float* f)
	{
		if constexpr (sizeof(T) == 2 && V % 2 == 0)
		{
			__half2* e = reinterpret_cast<__half2*>(&bits);
#pragma unroll
			for (int i = 0; i < V / 2; ++i) e[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
		}
		else
		{
			T* e = reinterpret_cast<T*>(&bits);
#pragma unroll
			for (int i = 0; i < V; ++i) e[i] = Cvt<T>::from_f32(f[i]);
		}
	}
};

}  // namespace b200
