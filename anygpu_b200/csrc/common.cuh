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

// Launch check that does not synchronise.
#define B200_LAUNCH_CHECK() B200_CUDA_TRY(cudaGetLastError())

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline int64_t cdiv(int64_t a, int64_t b) { return (a + b - 1) / b; }
inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

constexpr int kNumSMs = 148;  // B200: 2 dies x 74 SMs

// Device-side error word set by bounded waits (0 = none).
uint32_t* device_error_word();

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
__device__ __forceinline__ float silu_f32(float v) { return __fdividef(v, 1.0f + __expf(-v)); }

// torch softplus (beta 1, threshold 20), as F.softplus in scripts/zamba2/mamba_chunk_scan_comb.py:45.
__device__ __forceinline__ float softplus_f32(float v) { return v > 20.f ? v : log1pf(expf(v)); }

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
