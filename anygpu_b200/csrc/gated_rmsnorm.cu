// Fused gated RMSNorm: y = (x * silu(z)) * rsqrt(mean(g^2) + eps) * w in one pass over x and z.
// Stands in for the silu -> mul -> rms_norm chain of tensor_zamba_gated_rmsnorm
// (srcs/models/zamba2/zamba_gated_rmsnorm.hpp:9-23): 3 launches / 8 tensor passes there, 2 reads + 1 write here.
// HBM-bound: one CTA per (row, group); the gated values stay in registers between the statistic and the scaling.
#include "common.cuh"

namespace b200 {

constexpr int kNormCache = 4;  // 16-byte vectors cached per thread

template <typename T> struct NV;
template <> struct NV<__half>
{
	static constexpr int E = 8;
	static __device__ __forceinline__ void load(const __half* p, float* f) { unpack8(*reinterpret_cast<const Half8*>(p), f); }
	static __device__ __forceinline__ void store(__half* p, const float* f) { *reinterpret_cast<Half8*>(p) = pack8(f); }
};
template <> struct NV<float>
{
	static constexpr int E = 4;
	static __device__ __forceinline__ void load(const float* p, float* f)
	{
		const float4 v = *reinterpret_cast<const float4*>(p);
		f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
	}
	static __device__ __forceinline__ void store(float* p, const float* f)
	{
		*reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
	}
};

template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* red)
{
	v = warp_sum(v);
	const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
	if (lane == 0) red[wid] = v;
	__syncthreads();
	float t = (lane < THREADS / 32) ? red[lane] : 0.f;
	t = warp_sum(t);
	return t;  // identical in every thread of every warp
}

// VEC: 16-byte vectors (rows and group starts 16-byte aligned). CACHED: the group fits the register cache.
template <typename T, bool CACHED, int kNormThreads>
__global__ void __launch_bounds__(kNormThreads) gated_rmsnorm_vec_kernel(const T* x, int64_t xs,
	const T* __restrict__ z, int64_t zs, const T* __restrict__ w, T* y /* may alias x */, int64_t ys, int gsize, int ngroups, float eps,
	int ONCE /* x and z are dead after this kernel: their lines are marked first to leave L2 */)
{
	constexpr int E = NV<T>::E;
	__shared__ float red[kNormThreads / 32];
	const int64_t row = blockIdx.x / ngroups;
	const int grp = static_cast<int>(blockIdx.x - row * ngroups);
	const T* xr = x + row * xs + static_cast<int64_t>(grp) * gsize;
	const T* zr = z + row * zs + static_cast<int64_t>(grp) * gsize;
	const T* wr = w + static_cast<int64_t>(grp) * gsize;
	T* yr = y + row * ys + static_cast<int64_t>(grp) * gsize;
	const int nvec = gsize / E;

	float g[CACHED ? kNormCache : 1][E];
	float ss = 0.f;
	if constexpr (CACHED)
	{
		// every 16-byte vector of x and z this thread will touch is requested before the first one is used: one memory round
		// trip per row instead of one per vector
		Pack<T, E> rx[kNormCache], rz[kNormCache];
#pragma unroll
		for (int it = 0; it < kNormCache; ++it)
		{
			const int i = threadIdx.x + it * kNormThreads;
			if (i < nvec)
			{
				if (ONCE) { rx[it].load_pinned_once(xr + i * E); rz[it].load_pinned_once(zr + i * E); }
				else { rx[it].load_pinned(xr + i * E); rz[it].load_pinned(zr + i * E); }
			}
		}
#pragma unroll
		for (int it = 0; it < kNormCache; ++it)
		{
			const int i = threadIdx.x + it * kNormThreads;
			if (i < nvec)
			{
				float xv[E], zv[E];
				rx[it].unpack(xv);
				rz[it].unpack(zv);
#pragma unroll
				for (int e = 0; e < E; ++e)
				{
					const float gv = xv[e] * silu_f32(zv[e]);
					g[it][e] = gv;
					ss += gv * gv;
				}
			}
		}
	}
	else
	{
		for (int i = threadIdx.x; i < nvec; i += kNormThreads)
		{
			float xv[E], zv[E];
			NV<T>::load(xr + i * E, xv);
			NV<T>::load(zr + i * E, zv);
#pragma unroll
			for (int e = 0; e < E; ++e)
			{
				const float gv = xv[e] * silu_f32(zv[e]);
				ss += gv * gv;
			}
		}
	}
	const float total = block_sum<kNormThreads>(ss, red);
	const float scale = rsqrtf(total / static_cast<float>(gsize) + eps);

	if constexpr (CACHED)
	{
#pragma unroll
		for (int it = 0; it < kNormCache; ++it)
		{
			const int i = threadIdx.x + it * kNormThreads;
			if (i < nvec)
			{
				float wv[E], o[E];
				NV<T>::load(wr + i * E, wv);
#pragma unroll
				for (int e = 0; e < E; ++e) o[e] = g[it][e] * scale * wv[e];
				NV<T>::store(yr + i * E, o);
			}
		}
	}
	else
	{
		for (int i = threadIdx.x; i < nvec; i += kNormThreads)
		{
			float xv[E], zv[E], wv[E], o[E];
			NV<T>::load(xr + i * E, xv);
			NV<T>::load(zr + i * E, zv);
			NV<T>::load(wr + i * E, wv);
#pragma unroll
			for (int e = 0; e < E; ++e) o[e] = xv[e] * silu_f32(zv[e]) * scale * wv[e];
			NV<T>::store(yr + i * E, o);
		}
	}
}

// Any alignment / size.
template <typename T, int kNormThreads>
__global__ void __launch_bounds__(kNormThreads) gated_rmsnorm_scalar_kernel(const T* x, int64_t xs,
	const T* __restrict__ z, int64_t zs, const T* __restrict__ w, T* y /* may alias x */, int64_t ys, int gsize, int ngroups, float eps)
{
	__shared__ float red[kNormThreads / 32];
	const int64_t row = blockIdx.x / ngroups;
	const int grp = static_cast<int>(blockIdx.x - row * ngroups);
	const T* xr = x + row * xs + static_cast<int64_t>(grp) * gsize;
	const T* zr = z + row * zs + static_cast<int64_t>(grp) * gsize;
	const T* wr = w + static_cast<int64_t>(grp) * gsize;
	T* yr = y + row * ys + static_cast<int64_t>(grp) * gsize;
	float ss = 0.f;
	for (int i = threadIdx.x; i < gsize; i += kNormThreads)
	{
		const float gv = ldf(xr + i) * silu_f32(ldf(zr + i));
		ss += gv * gv;
	}
	const float total = block_sum<kNormThreads>(ss, red);
	const float scale = rsqrtf(total / static_cast<float>(gsize) + eps);
	for (int i = threadIdx.x; i < gsize; i += kNormThreads)
	{
		const float gv = ldf(xr + i) * silu_f32(ldf(zr + i));
		stf(yr + i, gv * scale * ldf(wr + i));
	}
}

// ---- tensor-parallel split of the gated RMSNorm --------------------------------------------------------------------
// When d_inner is sharded over ranks, the statistic mean(g^2) spans ranks. The normalisation factor is one scalar per
// token, so it commutes with the out_proj that follows: each rank emits g*w un-normalised together with its partial
// sum of squares; after the all-reduce of (out_proj partials, sums of squares) one row scaling finishes the job.
template <typename T>
__global__ void __launch_bounds__(128) gated_mul_sumsq_kernel(const T* x, int64_t xs, const T* __restrict__ z, int64_t zs,
	const T* __restrict__ w, T* y /* may alias x */, int64_t ys, float* __restrict__ sumsq, int d)
{
	__shared__ float red[4];
	const int64_t row = blockIdx.x;
	const T* xr = x + row * xs;
	const T* zr = z + row * zs;
	T* yr = y + row * ys;
	float ss = 0.f;
	for (int i = threadIdx.x; i < d; i += 128)
	{
		const float gv = ldf(xr + i) * silu_f32(ldf(zr + i));
		ss += gv * gv;
		stf(yr + i, gv * ldf(w + i));
	}
	const float total = block_sum<128>(ss, red);
	if (threadIdx.x == 0) sumsq[row] = total;
}

// The same with 16-byte vectors (rows, w and d aligned to them): up to kNormCache vectors per thread requested up front.
template <typename T>
__global__ void __launch_bounds__(128) gated_mul_sumsq_vec_kernel(const T* x, int64_t xs, const T* __restrict__ z, int64_t zs,
	const T* __restrict__ w, T* y /* may alias x */, int64_t ys, float* __restrict__ sumsq, int d)
{
	constexpr int E = NV<T>::E;
	__shared__ float red[4];
	const int64_t row = blockIdx.x;
	const T* xr = x + row * xs;
	const T* zr = z + row * zs;
	T* yr = y + row * ys;
	const int nvec = d / E;
	float ss = 0.f;
	for (int i0 = threadIdx.x; i0 < nvec; i0 += kNormCache * 128)
	{
		Pack<T, E> rx[kNormCache], rz[kNormCache];
#pragma unroll
		for (int it = 0; it < kNormCache; ++it)
		{
			const int i = i0 + it * 128;
			if (i < nvec)
			{
				rx[it].load_pinned(xr + i * E);
				rz[it].load_pinned(zr + i * E);
			}
		}
#pragma unroll
		for (int it = 0; it < kNormCache; ++it)
		{
			const int i = i0 + it * 128;
			if (i < nvec)
			{
				float xv[E], zv[E], wv[E], o[E];
				rx[it].unpack(xv);
				rz[it].unpack(zv);
				NV<T>::load(w + i * E, wv);
#pragma unroll
				for (int e = 0; e < E; ++e)
				{
					const float gv = xv[e] * silu_f32(zv[e]);
					ss += gv * gv;
					o[e] = gv * wv[e];
				}
				NV<T>::store(yr + i * E, o);
			}
		}
	}
	const float total = block_sum<128>(ss, red);
	if (threadIdx.x == 0) sumsq[row] = total;
}

template <typename T>
__global__ void __launch_bounds__(256) row_scale_rsqrt_kernel(T* __restrict__ out, int64_t ld, const float* __restrict__ sumsq,
	int64_t rows, int cols, float inv_d, float eps)
{
	const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
	if (i >= rows * cols) return;
	const int64_t r = i / cols;
	const int c = static_cast<int>(i - r * cols);
	T* p = out + r * ld + c;
	stf(p, ldf(p) * rsqrtf(sumsq[r] * inv_d + eps));
}

// The same with 16-byte vectors: grid (vector blocks of a row, rows), no division.
template <typename T>
__global__ void __launch_bounds__(256) row_scale_rsqrt_vec_kernel(T* __restrict__ out, int64_t ld, const float* __restrict__ sumsq,
	int cols, float inv_d, float eps)
{
	constexpr int E = NV<T>::E;
	const int c = (blockIdx.x * blockDim.x + threadIdx.x) * E;
	if (c >= cols) return;
	const int64_t r = blockIdx.y + static_cast<int64_t>(blockIdx.z) * gridDim.y;
	const float sc = rsqrtf(sumsq[r] * inv_d + eps);
	T* p = out + r * ld + c;
	float v[E];
	NV<T>::load(p, v);
#pragma unroll
	for (int e = 0; e < E; ++e) v[e] *= sc;
	NV<T>::store(p, v);
}

// ---- plain RMSNorm (the input norm of the decoder layer around the mixer) ----------------------------------------------
// y = x * rsqrt(mean(x^2) + eps) * (w + delta), tensor_rms_norm over the last axis (srcs/ops/norm_ops.hpp:134-191; delta = 1
// for its zero_centered flag). One CTA per row, the row cached in registers between the statistic and the scaling when it fits.
template <typename T, int THREADS, int CACHE>
__global__ void __launch_bounds__(THREADS) rms_norm_vec_kernel(const T* __restrict__ x, int64_t xs, const T* __restrict__ w,
	T* __restrict__ y, int64_t ys, int d, float eps, float delta)
{
	constexpr int E = NV<T>::E;
	__shared__ float red[THREADS / 32];
	const int64_t row = blockIdx.x;
	const T* xr = x + row * xs;
	T* yr = y + row * ys;
	const int nvec = d / E;
	float v[CACHE][E], wv[CACHE][E];
	float ss = 0.f;
	Pack<T, E> rx[CACHE];  // all cached vectors of the row are requested before the first is used
#pragma unroll
	for (int it = 0; it < CACHE; ++it)
	{
		const int i = threadIdx.x + it * THREADS;
		if (i < nvec) rx[it].load_pinned(xr + i * E);
	}
#pragma unroll
	for (int it = 0; it < CACHE; ++it)
	{
		const int i = threadIdx.x + it * THREADS;
		if (i < nvec)
		{
			rx[it].unpack(v[it]);
			NV<T>::load(w + i * E, wv[it]);
#pragma unroll
			for (int e = 0; e < E; ++e) ss += v[it][e] * v[it][e];
		}
	}
	for (int i = threadIdx.x + CACHE * THREADS; i < nvec; i += THREADS)  // rows longer than the cache: second pass below
	{
		float t[E];
		NV<T>::load(xr + i * E, t);
#pragma unroll
		for (int e = 0; e < E; ++e) ss += t[e] * t[e];
	}
	const float scale = rsqrtf(block_sum<THREADS>(ss, red) / static_cast<float>(d) + eps);
#pragma unroll
	for (int it = 0; it < CACHE; ++it)
	{
		const int i = threadIdx.x + it * THREADS;
		if (i < nvec)
		{
			float o[E];
#pragma unroll
			for (int e = 0; e < E; ++e) o[e] = v[it][e] * scale * (wv[it][e] + delta);
			NV<T>::store(yr + i * E, o);
		}
	}
	for (int i = threadIdx.x + CACHE * THREADS; i < nvec; i += THREADS)
	{
		float t[E], wt[E], o[E];
		NV<T>::load(xr + i * E, t);
		NV<T>::load(w + i * E, wt);
#pragma unroll
		for (int e = 0; e < E; ++e) o[e] = t[e] * scale * (wt[e] + delta);
		NV<T>::store(yr + i * E, o);
	}
}

template <typename T>
__global__ void __launch_bounds__(256) rms_norm_scalar_kernel(const T* __restrict__ x, int64_t xs, const T* __restrict__ w,
	T* __restrict__ y, int64_t ys, int d, float eps, float delta)
{
	__shared__ float red[8];
	const int64_t row = blockIdx.x;
	const T* xr = x + row * xs;
	T* yr = y + row * ys;
	float ss = 0.f;
	for (int i = threadIdx.x; i < d; i += 256)
	{
		const float t = ldf(xr + i);
		ss += t * t;
	}
	const float scale = rsqrtf(block_sum<256>(ss, red) / static_cast<float>(d) + eps);
	for (int i = threadIdx.x; i < d; i += 256) stf(yr + i, ldf(xr + i) * scale * (ldf(w + i) + delta));
}

template <typename T>
static int rms_norm(const void* xv, int64_t xs, const void* wv, void* yv, int64_t ys, int64_t rows, int64_t d, float eps, float delta,
	cudaStream_t st)
{
	constexpr int E = NV<T>::E;
	const T* x = static_cast<const T*>(xv);
	const T* w = static_cast<const T*>(wv);
	T* y = static_cast<T*>(yv);
	if (rows > 0x7fffffffLL || d > 0x7fffffffLL) return B200_ERR_UNSUPPORTED;
	const unsigned g = static_cast<unsigned>(rows);
	const int dd = static_cast<int>(d);
	const bool vec = aligned16(x) && aligned16(w) && aligned16(y) && xs % E == 0 && ys % E == 0 && d % E == 0;
	if (!vec)
		rms_norm_scalar_kernel<T><<<g, 256, 0, st>>>(x, xs, w, y, ys, dd, eps, delta);
	else if (d / E <= 2 * 128)
		rms_norm_vec_kernel<T, 128, 2><<<g, 128, 0, st>>>(x, xs, w, y, ys, dd, eps, delta);
	else
		rms_norm_vec_kernel<T, 256, 2><<<g, 256, 0, st>>>(x, xs, w, y, ys, dd, eps, delta);
	B200_LAUNCH_CHECK();
	return B200_OK;
}

template <typename T>
static int gated_rmsnorm(const void* xv, int64_t xs, const void* zv, int64_t zs, const void* wv, void* yv, int64_t ys,
	int64_t rows, int64_t d, int64_t gsize, float eps, cudaStream_t st, int once = 0)
{
	constexpr int E = NV<T>::E;
	const T* x = static_cast<const T*>(xv);
	const T* z = static_cast<const T*>(zv);
	const T* w = static_cast<const T*>(wv);
	T* y = static_cast<T*>(yv);
	const int ngroups = static_cast<int>(d / gsize);
	const int64_t blocks = rows * ngroups;
	if (blocks > 0x7fffffffLL || gsize > 0x7fffffffLL) return B200_ERR_UNSUPPORTED;
	const unsigned g = static_cast<unsigned>(blocks);
	const int gs = static_cast<int>(gsize);
	const bool vec = aligned16(x) && aligned16(z) && aligned16(w) && aligned16(y) && xs % E == 0 && zs % E == 0 && ys % E == 0 &&
		gsize % E == 0;
	// smallest CTA whose register cache holds the group: more CTAs in flight per SM, shorter reduction
	if (!vec)
		gated_rmsnorm_scalar_kernel<T, 256><<<g, 256, 0, st>>>(x, xs, z, zs, w, y, ys, gs, ngroups, eps);
	else if (gsize / E <= kNormCache * 128)
		gated_rmsnorm_vec_kernel<T, true, 128><<<g, 128, 0, st>>>(x, xs, z, zs, w, y, ys, gs, ngroups, eps, once);
	else if (gsize / E <= kNormCache * 256)
		gated_rmsnorm_vec_kernel<T, true, 256><<<g, 256, 0, st>>>(x, xs, z, zs, w, y, ys, gs, ngroups, eps, once);
	else
		gated_rmsnorm_vec_kernel<T, false, 256><<<g, 256, 0, st>>>(x, xs, z, zs, w, y, ys, gs, ngroups, eps, once);
	B200_LAUNCH_CHECK();
	return B200_OK;
}

int gated_mul_sumsq(int dtype, const void* x, int64_t xs, const void* z, int64_t zs, const void* w, void* y, int64_t ys,
	float* sumsq, int64_t rows, int64_t d, cudaStream_t st)
{
	if (rows > 0x7fffffffLL || d > 0x7fffffffLL) return B200_ERR_UNSUPPORTED;
	const unsigned g = static_cast<unsigned>(rows);
	const size_t esz = dtype == B200_F16 ? 2 : 4;
	const int64_t ev = 16 / static_cast<int64_t>(esz);
	if (d % ev == 0 && xs % ev == 0 && zs % ev == 0 && ys % ev == 0 && aligned16(x) && aligned16(z) && aligned16(w) && aligned16(y))
	{
		if (dtype == B200_F16)
			gated_mul_sumsq_vec_kernel<__half><<<g, 128, 0, st>>>(static_cast<const __half*>(x), xs, static_cast<const __half*>(z), zs,
				static_cast<const __half*>(w), static_cast<__half*>(y), ys, sumsq, static_cast<int>(d));
		else
			gated_mul_sumsq_vec_kernel<float><<<g, 128, 0, st>>>(static_cast<const float*>(x), xs, static_cast<const float*>(z), zs,
				static_cast<const float*>(w), static_cast<float*>(y), ys, sumsq, static_cast<int>(d));
		B200_LAUNCH_CHECK();
		return B200_OK;
	}
	if (dtype == B200_F16)
		gated_mul_sumsq_kernel<__half><<<g, 128, 0, st>>>(static_cast<const __half*>(x), xs, static_cast<const __half*>(z), zs,
			static_cast<const __half*>(w), static_cast<__half*>(y), ys, sumsq, static_cast<int>(d));
	else
		gated_mul_sumsq_kernel<float><<<g, 128, 0, st>>>(static_cast<const float*>(x), xs, static_cast<const float*>(z), zs,
			static_cast<const float*>(w), static_cast<float*>(y), ys, sumsq, static_cast<int>(d));
	B200_LAUNCH_CHECK();
	return B200_OK;
}

int row_scale_rsqrt(int dtype, void* out, int64_t ld, const float* sumsq, int64_t rows, int64_t cols, float inv_d, float eps,
	cudaStream_t st)
{
	{
		const int64_t ev = dtype == B200_F16 ? 8 : 4;
		// rows as grid y * z (z > 1 only beyond 65535 rows, which must then split evenly)
		int64_t gy = rows, gz = 1;
		while (gy > 65535 && gz < 65535) { gz *= 2; gy = rows / gz; }
		if (cols % ev == 0 && ld % ev == 0 && aligned16(out) && cols <= 0x7fffffffLL && gy * gz == rows && gy <= 65535 && rows > 0 &&
			(dtype == B200_F16 || dtype == B200_F32))
		{
			const dim3 g(static_cast<unsigned>(cdiv(cols / ev, 256)), static_cast<unsigned>(gy), static_cast<unsigned>(gz));
			if (dtype == B200_F16)
				row_scale_rsqrt_vec_kernel<__half><<<g, 256, 0, st>>>(static_cast<__half*>(out), ld, sumsq, static_cast<int>(cols), inv_d, eps);
			else
				row_scale_rsqrt_vec_kernel<float><<<g, 256, 0, st>>>(static_cast<float*>(out), ld, sumsq, static_cast<int>(cols), inv_d, eps);
			B200_LAUNCH_CHECK();
			return B200_OK;
		}
	}
	const int64_t blocks = cdiv(rows * cols, 256);
	if (blocks > 0x7fffffffLL || cols > 0x7fffffffLL) return B200_ERR_UNSUPPORTED;
	if (dtype == B200_F16)
		row_scale_rsqrt_kernel<__half><<<static_cast<unsigned>(blocks), 256, 0, st>>>(static_cast<__half*>(out), ld, sumsq, rows,
			static_cast<int>(cols), inv_d, eps);
	else
		row_scale_rsqrt_kernel<float><<<static_cast<unsigned>(blocks), 256, 0, st>>>(static_cast<float*>(out), ld, sumsq, rows,
			static_cast<int>(cols), inv_d, eps);
	B200_LAUNCH_CHECK();
	return B200_OK;
}

// The gated norm inside the prefill mixer: its inputs (the scan's y, read in place, and the z columns of the in_proj output) are
// not read again, so they are loaded with an evict-first L2 policy and the output, which out_proj reads next, is what stays in L2
// (8192 x 4096: 36.2 -> 34.9 us).
int gated_rmsnorm_last_use(int dtype, const void* x, int64_t xs, const void* z, int64_t zs, const void* w, void* y, int64_t ys,
	int64_t rows, int64_t d, int64_t group_size, float eps, cudaStream_t st)
{
	if (group_size == 0) group_size = d;
	if (rows <= 0) return B200_OK;
	if (dtype == B200_F16) return gated_rmsnorm<__half>(x, xs, z, zs, w, y, ys, rows, d, group_size, eps, st, 1);
	return gated_rmsnorm<float>(x, xs, z, zs, w, y, ys, rows, d, group_size, eps, st, 1);
}

}  // namespace b200

using namespace b200;

extern "C" int b200_gated_rmsnorm(int dtype, const void* x, int64_t x_stride, const void* z, int64_t z_stride, const void* w,
	void* y, int64_t y_stride, int64_t rows, int64_t d, int64_t group_size, float eps, void* stream)
{
	if (!x || !z || !w || !y) return B200_ERR_NULL;
	if (group_size == 0) group_size = d;
	if (rows < 0 || d <= 0 || group_size <= 0 || d % group_size != 0 || x_stride < d || z_stride < d || y_stride < d)
		return B200_ERR_BAD_SHAPE;
	if (rows == 0) return B200_OK;
	cudaStream_t st = static_cast<cudaStream_t>(stream);
	if (dtype == B200_F16) return gated_rmsnorm<__half>(x, x_stride, z, z_stride, w, y, y_stride, rows, d, group_size, eps, st);
	if (dtype == B200_F32) return gated_rmsnorm<float>(x, x_stride, z, z_stride, w, y, y_stride, rows, d, group_size, eps, st);
	return B200_ERR_UNSUPPORTED;
}

extern "C" int b200_rms_norm(int dtype, const void* x, int64_t x_stride, const void* w, void* y, int64_t y_stride, int64_t rows,
	int64_t dim, float eps, int zero_centered, void* stream)
{
	if (!x || !w || !y) return B200_ERR_NULL;
	if (rows < 0 || dim <= 0 || x_stride < dim || y_stride < dim) return B200_ERR_BAD_SHAPE;
	if (rows == 0) return B200_OK;
	cudaStream_t st = static_cast<cudaStream_t>(stream);
	const float delta = zero_centered ? 1.f : 0.f;
	if (dtype == B200_F16) return rms_norm<__half>(x, x_stride, w, y, y_stride, rows, dim, eps, delta, st);
	if (dtype == B200_F32) return rms_norm<float>(x, x_stride, w, y, y_stride, rows, dim, eps, delta, st);
	return B200_ERR_UNSUPPORTED;
}
