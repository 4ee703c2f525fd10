// Depthwise causal conv1d + bias + SiLU for the Mamba2 mixer: full-sequence kernels in both tensor layouts and
// the single-token conv_state update. HBM-bound: every element is read once and written once through 128-bit
// accesses; the (width-1)-element halo comes from the neighbouring lane by warp shuffle (or a cached re-read at
// warp boundaries). fp32 accumulation in the tap order of anyGPU's CPU operator
// (srcs/fused/causal_conv1d.hpp:55-84): taps oldest-first, bias last, then x / (1 + exp(-x)).
#include "conv_dt_bodies.cuh"

namespace b200 {

constexpr int kMaxWidth = 4;  // same limit as anyGPU's CUDA operator (srcs/fused/causal_conv1d.hpp:100)

template <typename T> struct Vec16;
template <> struct Vec16<__half>
{
	static constexpr int E = 8;
	static __device__ __forceinline__ void load(const __half* p, float* f)
	{
		Half8 v = *reinterpret_cast<const Half8*>(p);
		unpack8(v, f);
	}
	static __device__ __forceinline__ void store(__half* p, const float* f) { *reinterpret_cast<Half8*>(p) = pack8(f); }
};
template <> struct Vec16<float>
{
	static constexpr int E = 4;
	static __device__ __forceinline__ void load(const float* p, float* f)
	{
		float4 v = *reinterpret_cast<const float4*>(p);
		f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
	}
	static __device__ __forceinline__ void store(float* p, const float* f)
	{
		*reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
	}
};

// ---- (batch, dims, seq_len) layout: sequence contiguous -----------------------------------------------------
// One thread owns NV consecutive 16-byte vectors of one row. A row is S elements; S % (E*NV) == 0.
template <typename T, int NV, int W>
__global__ void __launch_bounds__(256) conv1d_seq_vec_kernel(const T* __restrict__ x, const T* __restrict__ w,
	const T* __restrict__ bias, T* __restrict__ y, int vec_per_row /* S / (E*NV) */, unsigned dims)
{
	// grid: x = blocks along one row, y = row (batch * dims + channel); no 64-bit divisions on the hot path
	constexpr int E = Vec16<T>::E;
	constexpr int EPT = E * NV;
	const unsigned row = blockIdx.y + blockIdx.z * 65535u;
	const int j = static_cast<int>(blockIdx.x * blockDim.x + threadIdx.x);
	const bool active = j < vec_per_row;
	const int64_t base = static_cast<int64_t>(row) * (static_cast<int64_t>(vec_per_row) * EPT) + static_cast<int64_t>(j) * EPT;

	// lane 0 cannot get its halo from a neighbour: fetch it first so that it does not queue behind the main loads
	const int lane = threadIdx.x & 31;
	float g0 = 0.f, g1 = 0.f, g2 = 0.f;
	if (active && lane == 0 && j > 0)
	{
		g0 = ldf(x + base - 3);
		g1 = ldf(x + base - 2);
		g2 = ldf(x + base - 1);
	}
	float v[EPT + 3];  // v[0..2] = halo, v[3..] = own elements
	if (active)
	{
#pragma unroll
		for (int i = 0; i < NV; ++i) Vec16<T>::load(x + base + i * E, v + 3 + i * E);
	}
	else
	{
#pragma unroll
		for (int i = 0; i < EPT; ++i) v[3 + i] = 0.f;
	}
	// halo: last three elements of the previous lane's run (same row when j > 0)
	float h0 = __shfl_up_sync(0xffffffffu, v[EPT], 1);
	float h1 = __shfl_up_sync(0xffffffffu, v[EPT + 1], 1);
	float h2 = __shfl_up_sync(0xffffffffu, v[EPT + 2], 1);
	if (!active) return;
	if (j == 0)
	{
		h0 = h1 = h2 = 0.f;  // zero left padding
	}
	else if (lane == 0)
	{
		h0 = g0; h1 = g1; h2 = g2;
	}
	v[0] = h0; v[1] = h1; v[2] = h2;

	const unsigned d = row % dims;
	float wt[W];
#pragma unroll
	for (int k = 0; k < W; ++k) wt[k] = ldf(w + static_cast<int64_t>(d) * W + k);
	const float bs = ldf(bias + d);

	float out[EPT];
#pragma unroll
	for (int i = 0; i < EPT; ++i)
	{
		float acc = 0.f;
#pragma unroll
		for (int k = 0; k < W; ++k) acc += wt[k] * v[3 + i + k - (W - 1)];
		acc += bs;
		out[i] = silu_f32(acc);
	}
#pragma unroll
	for (int i = 0; i < NV; ++i) Vec16<T>::store(y + base + i * E, out + i * E);
}

// Width 4, long rows: one CTA per row, a thread owns NVI 16-byte vectors that lie blockDim.x vectors apart, so that every
// load and store instruction of a warp covers 512 contiguous bytes and all NVI loads of a thread are in flight together. The
// three elements before a vector come from the neighbouring lane by shuffle; lane 0 of a warp reads the 4 elements in front of its
// vector instead (vector 0 of a row sees the zero padding). The per-thread overhead (weights, addressing) is paid once per
// NVI * E outputs.
template <typename T, int NVI>
__global__ void __launch_bounds__(256) conv1d_seq_w4_kernel(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ bias,
	T* __restrict__ y, int vec_per_row /* S / E, a multiple of blockDim.x * NVI */, unsigned dims)
{
	constexpr int E = Vec16<T>::E;
	constexpr int HV = 4;  // elements fetched in front of a vector by lane 0 (8 or 16 bytes, aligned like the vector); 3 are used
	const unsigned row = blockIdx.y + blockIdx.z * 65535u;
	const int lane = threadIdx.x & 31;
	const int64_t rbase = static_cast<int64_t>(row) * (static_cast<int64_t>(vec_per_row) * E);
	const int v0 = blockIdx.x * (blockDim.x * NVI) + threadIdx.x;

	Pack<T, E> raw[NVI];
	Pack<T, HV> head[NVI];
#pragma unroll
	for (int i = 0; i < NVI; ++i) raw[i].load_pinned(x + rbase + static_cast<int64_t>(v0 + i * static_cast<int>(blockDim.x)) * E);
	if (lane == 0)
	{
#pragma unroll
		for (int i = 0; i < NVI; ++i)
		{
			const int v = v0 + i * static_cast<int>(blockDim.x);
			if (v > 0) head[i].load_pinned(x + rbase + static_cast<int64_t>(v) * E - HV);
		}
	}
	const unsigned d = row % dims;
	Pack<T, 4> wp;
	wp.load(w + static_cast<int64_t>(d) * 4);
	float wt[4];
	wp.unpack(wt);
	const float bs = ldf(bias + d);

#pragma unroll
	for (int i = 0; i < NVI; ++i)
	{
		const int v = v0 + i * static_cast<int>(blockDim.x);
		float f[E + 3];
		raw[i].unpack(f + 3);
		float h0 = __shfl_up_sync(0xffffffffu, f[E], 1);
		float h1 = __shfl_up_sync(0xffffffffu, f[E + 1], 1);
		float h2 = __shfl_up_sync(0xffffffffu, f[E + 2], 1);
		if (lane == 0)
		{
			h0 = h1 = h2 = 0.f;  // zero left padding in front of the row
			if (v > 0)
			{
				float hf[HV];
				head[i].unpack(hf);
				h0 = hf[HV - 3]; h1 = hf[HV - 2]; h2 = hf[HV - 1];
			}
		}
		f[0] = h0; f[1] = h1; f[2] = h2;
		float out[E];
#pragma unroll
		for (int e = 0; e < E; ++e)
		{
			float acc = 0.f;  // taps oldest first, bias last
#pragma unroll
			for (int k = 0; k < 4; ++k) acc += wt[k] * f[e + k];
			acc += bs;
			out[e] = silu_f32(acc);
		}
		Pack<T, E> o;
		o.pack(out);
		o.store(y + rbase + static_cast<int64_t>(v) * E);
	}
}

// Any shape: one thread per output element.
template <typename T>
__global__ void __launch_bounds__(256) conv1d_seq_scalar_kernel(const T* __restrict__ x, const T* __restrict__ w,
	const T* __restrict__ bias, T* __restrict__ y, int64_t total, int64_t S, int64_t dims, int W)
{
	const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
	if (i >= total) return;
	const int64_t row = i / S;
	const int64_t s = i - row * S;
	const int64_t d = row % dims;
	float acc = 0.f;
	for (int k = 0; k < W; ++k)
	{
		const int64_t delta = s + k - (W - 1);
		if (delta >= 0) acc += ldf(w + d * W + k) * ldf(x + row * S + delta);
	}
	acc += ldf(bias + d);
	stf(y + i, silu_f32(acc));
}

// ---- token-major layout: channels contiguous, rows strided ---------------------------------------------------
// One thread owns V consecutive channels (one 8-byte access for f16, 16-byte for f32, or a single element) and TL
// consecutive tokens. All TL + W - 1 row fragments are loaded before the first use, so a thread keeps TL + W - 1
// loads in flight while its register footprint stays small enough for ~28 resident warps per SM.
template <typename T, int V, int W, int TL>
__global__ void __launch_bounds__(128, 7) conv1d_tok_kernel(const T* __restrict__ x, int64_t xs, const T* __restrict__ w,
	const T* __restrict__ bias, T* __restrict__ y, int64_t ys, const T* __restrict__ init, T* __restrict__ fin,
	int seqlen, int dims, unsigned cvec /* ceil(dims / V) */, unsigned nwork /* cvec * token blocks */)
{
	conv1d_tok_body<T, V, W, TL>(x, xs, w, bias, y, ys, init, fin, seqlen, dims, cvec, nwork, blockIdx.x, blockIdx.y);
}

// ---- decode: one token, rolling state ----------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) conv1d_update_kernel(const T* __restrict__ xt, int64_t xs, T* __restrict__ state,
	const T* __restrict__ w, const T* __restrict__ bias, T* __restrict__ yt, int64_t ys, int64_t batch, int64_t dims, int W)
{
	const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
	if (i >= batch * dims) return;
	const int64_t b = i / dims;
	const int64_t d = i - b * dims;
	const int SW = W - 1;
	T* st = state + i * SW;
	float s[kMaxWidth];
	for (int k = 0; k < SW; ++k) s[k] = ldf(st + k);
	const float xv = ldf(xt + b * xs + d);
	float acc = 0.f;
	for (int k = 0; k < SW; ++k) acc += ldf(w + d * W + k) * s[k];
	acc += ldf(w + d * W + SW) * xv;
	acc += ldf(bias + d);
	stf(yt + b * ys + d, silu_f32(acc));
	for (int k = 0; k + 1 < SW; ++k) stf(st + k, s[k + 1]);
	if (SW > 0) stf(st + SW - 1, xv);
}

// Width 4, 4 channels per thread: their 12 state values, 16 taps, 4 biases and 4 inputs are each contiguous, so the step is
// 9 vector loads and 4 vector stores per thread instead of 24 scalar accesses per channel; grid (channel quads, batch).
template <typename T>
__global__ void __launch_bounds__(128) conv1d_update_w4_kernel(const T* __restrict__ xt, int64_t xs, T* __restrict__ state,
	const T* __restrict__ w, const T* __restrict__ bias, T* __restrict__ yt, int64_t ys, int dims)
{
	const int d = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
	if (d >= dims) return;
	const int64_t b = blockIdx.y;
	T* st = state + (b * dims + d) * 3;
	Pack<T, 4> sv[3], wv[4], bv, xv;
#pragma unroll
	for (int i = 0; i < 3; ++i) sv[i].load(st + i * 4);
	xv.load(xt + b * xs + d);
#pragma unroll
	for (int c = 0; c < 4; ++c) wv[c].load(w + static_cast<int64_t>(d + c) * 4);
	bv.load(bias + d);
	float s[12], x[4], bs[4], y[4];
#pragma unroll
	for (int i = 0; i < 3; ++i) sv[i].unpack(s + i * 4);  // channel-major: s[c * 3 + k]
	xv.unpack(x);
	bv.unpack(bs);
#pragma unroll
	for (int c = 0; c < 4; ++c)
	{
		float wt[4];
		wv[c].unpack(wt);
		float acc = 0.f;  // taps oldest first, bias last
#pragma unroll
		for (int k = 0; k < 3; ++k) acc += wt[k] * s[c * 3 + k];
		acc += wt[3] * x[c];
		acc += bs[c];
		y[c] = silu_f32(acc);
		s[c * 3] = s[c * 3 + 1];
		s[c * 3 + 1] = s[c * 3 + 2];
		s[c * 3 + 2] = x[c];
	}
	Pack<T, 4> o;
	o.pack(y);
	o.store(yt + b * ys + d);
#pragma unroll
	for (int i = 0; i < 3; ++i)
	{
		sv[i].pack(s + i * 4);
		sv[i].store(st + i * 4);
	}
}

// ---- host launchers ----------------------------------------------------------------------------------------

template <typename T, int NV>
static int launch_seq_vec(const T* x, const T* w, const T* bias, T* y, int64_t rows, int64_t S, int64_t dims, int W,
	cudaStream_t st)
{
	constexpr int EPT = Vec16<T>::E * NV;
	const int vec_per_row = static_cast<int>(S / EPT);
	if (rows > 65535LL * 65535LL || dims > 0x7fffffffLL) return B200_ERR_UNSUPPORTED;
	const int threads = vec_per_row >= 256 ? 256 : (vec_per_row >= 128 ? 128 : (vec_per_row >= 64 ? 64 : 32));
	// rows = gy * gz exactly (gz > 1 only beyond 65535 rows, which must then be a multiple of 65535)
	unsigned gy = static_cast<unsigned>(rows), gz = 1;
	if (rows > 65535)
	{
		if (rows % 65535 != 0) return B200_ERR_UNSUPPORTED;
		gy = 65535u;
		gz = static_cast<unsigned>(rows / 65535);
	}
	const dim3 g(static_cast<unsigned>(cdiv(vec_per_row, threads)), gy, gz);
	const unsigned dm = static_cast<unsigned>(dims);
	switch (W)
	{
	case 1: conv1d_seq_vec_kernel<T, NV, 1><<<g, threads, 0, st>>>(x, w, bias, y, vec_per_row, dm); break;
	case 2: conv1d_seq_vec_kernel<T, NV, 2><<<g, threads, 0, st>>>(x, w, bias, y, vec_per_row, dm); break;
	case 3: conv1d_seq_vec_kernel<T, NV, 3><<<g, threads, 0, st>>>(x, w, bias, y, vec_per_row, dm); break;
	default: conv1d_seq_vec_kernel<T, NV, 4><<<g, threads, 0, st>>>(x, w, bias, y, vec_per_row, dm); break;
	}
	B200_LAUNCH_CHECK();
	return B200_OK;
}

template <typename T>
static int conv1d_seq(const void* xv, const void* wv, const void* bv, void* yv, int64_t batch, int64_t dims, int64_t S, int W,
	cudaStream_t st)
{
	const T* x = static_cast<const T*>(xv);
	const T* w = static_cast<const T*>(wv);
	const T* bias = static_cast<const T*>(bv);
	T* y = static_cast<T*>(yv);
	const int64_t rows = batch * dims;
	constexpr int E = Vec16<T>::E;
	const bool al = aligned16(x) && aligned16(y);
	const bool grid_ok = rows <= 65535 || rows % 65535 == 0;
	if (al && grid_ok && W == 4 && S % E == 0 && (reinterpret_cast<uintptr_t>(w) % (4 * sizeof(T))) == 0 &&
		dims <= 0x7fffffffLL)
	{
		// threads x vectors per thread that tile the row exactly; prefer 8 vectors per thread
		const int64_t vpr = S / E;
		int threads = 0, nvi = 0;
		// measured at 8 x 4224 rows of 4096 f16: 8 vectors per thread 103-105 us, 4 vectors 115-117 us, 2 vectors 107-111 us, 16 vectors
		// 133 us (130 registers)
		for (int t : { 64, 32, 128, 256 })
		{
			if (vpr % (t * 8) == 0) { threads = t; nvi = 8; break; }
		}
		if (!threads)
			for (int t : { 128, 256, 64, 32 })
			{
				if (vpr % (t * 4) == 0) { threads = t; nvi = 4; break; }
			}
		if (!threads)
			for (int t : { 256, 128, 64, 32 })
			{
				if (vpr % (t * 2) == 0) { threads = t; nvi = 2; break; }
			}
		if (threads)
		{
			unsigned gy = static_cast<unsigned>(rows), gz = 1;
			if (rows > 65535) { gy = 65535u; gz = static_cast<unsigned>(rows / 65535); }
			const dim3 g(static_cast<unsigned>(vpr / (threads * nvi)), gy, gz);
			if (nvi == 8) conv1d_seq_w4_kernel<T, 8><<<g, threads, 0, st>>>(x, w, bias, y, static_cast<int>(vpr), static_cast<unsigned>(dims));
			else if (nvi == 4) conv1d_seq_w4_kernel<T, 4><<<g, threads, 0, st>>>(x, w, bias, y, static_cast<int>(vpr), static_cast<unsigned>(dims));
			else conv1d_seq_w4_kernel<T, 2><<<g, threads, 0, st>>>(x, w, bias, y, static_cast<int>(vpr), static_cast<unsigned>(dims));
			B200_LAUNCH_CHECK();
			return B200_OK;
		}
	}
	if (al && grid_ok && S % (2 * E) == 0) return launch_seq_vec<T, 2>(x, w, bias, y, rows, S, dims, W, st);
	if (al && grid_ok && S % E == 0) return launch_seq_vec<T, 1>(x, w, bias, y, rows, S, dims, W, st);
	const int64_t total = rows * S;
	const int64_t blocks = cdiv(total, 256);
	if (blocks > 0x7fffffffLL) return B200_ERR_UNSUPPORTED;
	conv1d_seq_scalar_kernel<T><<<static_cast<unsigned>(blocks), 256, 0, st>>>(x, w, bias, y, total, S, dims, W);
	B200_LAUNCH_CHECK();
	return B200_OK;
}

template <typename T, int V>
static int launch_tok(const T* x, int64_t xs, const T* w, const T* bias, T* y, int64_t ys, const T* init, T* fin,
	int64_t batch, int64_t seqlen, int64_t dims, int W, cudaStream_t st)
{
	constexpr int TL = 8;
	const int64_t cvec = cdiv(dims, V);
	const int64_t nwork = cvec * cdiv(seqlen, TL);
	if (nwork > 0x7fffffffLL || batch > 65535 || seqlen > 0x7fffffffLL || dims > 0x7fffffffLL) return B200_ERR_UNSUPPORTED;
	const dim3 g(static_cast<unsigned>(cdiv(nwork, 128)), static_cast<unsigned>(batch));
	const int sl = static_cast<int>(seqlen), dm = static_cast<int>(dims);
	const unsigned cv = static_cast<unsigned>(cvec), nw = static_cast<unsigned>(nwork);
	switch (W)
	{
	case 1: conv1d_tok_kernel<T, V, 1, TL><<<g, 128, 0, st>>>(x, xs, w, bias, y, ys, init, fin, sl, dm, cv, nw); break;
	case 2: conv1d_tok_kernel<T, V, 2, TL><<<g, 128, 0, st>>>(x, xs, w, bias, y, ys, init, fin, sl, dm, cv, nw); break;
	case 3: conv1d_tok_kernel<T, V, 3, TL><<<g, 128, 0, st>>>(x, xs, w, bias, y, ys, init, fin, sl, dm, cv, nw); break;
	default: conv1d_tok_kernel<T, V, 4, TL><<<g, 128, 0, st>>>(x, xs, w, bias, y, ys, init, fin, sl, dm, cv, nw); break;
	}
	B200_LAUNCH_CHECK();
	return B200_OK;
}

template <typename T>
static int conv1d_tok(const void* xv, int64_t xs, const void* wv, const void* bv, void* yv, int64_t ys, const void* init,
	void* fin, int64_t batch, int64_t seqlen, int64_t dims, int W, cudaStream_t st)
{
	constexpr int V = 4;  // 8 bytes of f16 / 16 bytes of f32 per access
	const uintptr_t amask = V * sizeof(T) - 1;
	// the width-4 body also fetches the 4 taps of a channel and the 4 biases of a channel quad with one access each
	const bool wb_ok = W != 4 || ((reinterpret_cast<uintptr_t>(wv) & amask) == 0 && (reinterpret_cast<uintptr_t>(bv) & amask) == 0);
	const bool vec = (reinterpret_cast<uintptr_t>(xv) & amask) == 0 && (reinterpret_cast<uintptr_t>(yv) & amask) == 0 && xs % V == 0 &&
		ys % V == 0 && dims % V == 0 && wb_ok;
	if (vec)
		return launch_tok<T, V>(static_cast<const T*>(xv), xs, static_cast<const T*>(wv), static_cast<const T*>(bv),
			static_cast<T*>(yv), ys, static_cast<const T*>(init), static_cast<T*>(fin), batch, seqlen, dims, W, st);
	return launch_tok<T, 1>(static_cast<const T*>(xv), xs, static_cast<const T*>(wv), static_cast<const T*>(bv),
		static_cast<T*>(yv), ys, static_cast<const T*>(init), static_cast<T*>(fin), batch, seqlen, dims, W, st);
}

}  // namespace b200

using namespace b200;

extern "C" int b200_causal_conv1d(int dtype, const void* x, const void* w, const void* bias, void* y,
	int64_t batch, int64_t dims, int64_t seqlen, int width, void* stream)
{
	if (!x || !w || !bias || !y) return B200_ERR_NULL;
	if (batch < 0 || dims <= 0 || seqlen < 0 || width < 1 || width > kMaxWidth) return B200_ERR_BAD_SHAPE;
	if (batch == 0 || seqlen == 0) return B200_OK;
	cudaStream_t st = static_cast<cudaStream_t>(stream);
	if (dtype == B200_F16) return conv1d_seq<__half>(x, w, bias, y, batch, dims, seqlen, width, st);
	if (dtype == B200_F32) return conv1d_seq<float>(x, w, bias, y, batch, dims, seqlen, width, st);
	return B200_ERR_UNSUPPORTED;
}

extern "C" int b200_causal_conv1d_tokens(int dtype, const void* x, int64_t x_stride, const void* w, const void* bias,
	void* y, int64_t y_stride, const void* initial_state, void* final_state,
	int64_t batch, int64_t seqlen, int64_t dims, int width, void* stream)
{
	if (!x || !w || !bias || !y) return B200_ERR_NULL;
	if (batch < 0 || dims <= 0 || seqlen < 0 || width < 1 || width > kMaxWidth || x_stride < dims || y_stride < dims)
		return B200_ERR_BAD_SHAPE;
	if (batch == 0 || seqlen == 0) return B200_OK;
	cudaStream_t st = static_cast<cudaStream_t>(stream);
	if (dtype == B200_F16)
		return conv1d_tok<__half>(x, x_stride, w, bias, y, y_stride, initial_state, final_state, batch, seqlen, dims, width, st);
	if (dtype == B200_F32)
		return conv1d_tok<float>(x, x_stride, w, bias, y, y_stride, initial_state, final_state, batch, seqlen, dims, width, st);
	return B200_ERR_UNSUPPORTED;
}

extern "C" int b200_causal_conv1d_update(int dtype, const void* x_t, int64_t x_stride, void* conv_state, const void* w,
	const void* bias, void* y_t, int64_t y_stride, int64_t batch, int64_t dims, int width, void* stream)
{
	if (!x_t || !conv_state || !w || !bias || !y_t) return B200_ERR_NULL;
	if (batch < 0 || dims <= 0 || width < 1 || width > kMaxWidth || x_stride < dims || y_stride < dims) return B200_ERR_BAD_SHAPE;
	if (batch == 0) return B200_OK;
	cudaStream_t st = static_cast<cudaStream_t>(stream);
	const size_t vb = 4 * (dtype == B200_F16 ? 2 : 4);  // bytes of a 4-element vector
	auto al = [vb](const void* p) { return (reinterpret_cast<uintptr_t>(p) % vb) == 0; };
	if (width == 4 && dims % 4 == 0 && x_stride % 4 == 0 && y_stride % 4 == 0 && batch <= 65535 && dims <= 0x7fffffffLL && al(x_t) &&
		al(conv_state) && al(w) && al(bias) && al(y_t) && (dtype == B200_F16 || dtype == B200_F32))
	{
		const dim3 g(static_cast<unsigned>(cdiv(dims / 4, 128)), static_cast<unsigned>(batch));
		if (dtype == B200_F16)
			conv1d_update_w4_kernel<__half><<<g, 128, 0, st>>>(static_cast<const __half*>(x_t), x_stride, static_cast<__half*>(conv_state),
				static_cast<const __half*>(w), static_cast<const __half*>(bias), static_cast<__half*>(y_t), y_stride, static_cast<int>(dims));
		else
			conv1d_update_w4_kernel<float><<<g, 128, 0, st>>>(static_cast<const float*>(x_t), x_stride, static_cast<float*>(conv_state),
				static_cast<const float*>(w), static_cast<const float*>(bias), static_cast<float*>(y_t), y_stride, static_cast<int>(dims));
		B200_LAUNCH_CHECK();
		return B200_OK;
	}
	const unsigned blocks = static_cast<unsigned>(cdiv(batch * dims, 256));
	if (dtype == B200_F16)
		conv1d_update_kernel<__half><<<blocks, 256, 0, st>>>(static_cast<const __half*>(x_t), x_stride,
			static_cast<__half*>(conv_state), static_cast<const __half*>(w), static_cast<const __half*>(bias),
			static_cast<__half*>(y_t), y_stride, batch, dims, width);
	else if (dtype == B200_F32)
		conv1d_update_kernel<float><<<blocks, 256, 0, st>>>(static_cast<const float*>(x_t), x_stride,
			static_cast<float*>(conv_state), static_cast<const float*>(w), static_cast<const float*>(bias),
			static_cast<float*>(y_t), y_stride, batch, dims, width);
	else
		return B200_ERR_UNSUPPORTED;
	B200_LAUNCH_CHECK();
	return B200_OK;
}
