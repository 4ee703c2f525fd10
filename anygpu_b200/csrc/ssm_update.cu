// Single-token ssm_state recurrence for decode:
//   dt = softplus(dt_raw + dt_bias); h <- exp(dt*A) h + dt x (x) B; y = h.C + D x    per (batch, head).
// HBM-bound: the fp32 state [b,H,P,N] is read once and written once with 128-bit accesses (a 64-wide state row is
// 16 lanes x float4); everything else is noise next to it. The y reduction over N runs in warp shuffles.
#include "common.cuh"

namespace b200 {

// LPR lanes share one (b,h,p) row of N = 4*LPR states (LPR a power of two <= 32). A thread owns RPT rows, 256/LPR
// rows apart, and issues all of their 128-bit state loads before the first use, so that enough bytes are in flight
// per SM to cover HBM latency. B and C are read as one 8-byte (f16) or 16-byte (f32) vector per thread.
// GATE: the output is additionally gated and weighted for the RMSNorm that follows, y <- round_T(y) * silu(z) * norm_w, and the
// CTA's sum of (round_T(y) * silu(z))^2 goes to sumsq[b, h]; the consumer of y applies rsqrt(mean + eps) (a row scale commutes
// with the projection that follows the norm).
template <typename T, int LPR, int RPT, bool GATE = false>
__global__ void __launch_bounds__(256) ssm_update_vec_kernel(float* __restrict__ state, const T* __restrict__ x, int64_t xs,
	const T* __restrict__ dt, int64_t dts, const float* __restrict__ A, int a_is_log, const T* __restrict__ Bm, int64_t bs,
	const T* __restrict__ Cm, int64_t cs, const float* __restrict__ D, const float* __restrict__ dt_bias, T* __restrict__ y,
	int64_t ys, int H, int P, int G, int dt_softplus, const T* __restrict__ z = nullptr, int64_t zs = 0,
	const T* __restrict__ norm_w = nullptr, float* __restrict__ sumsq = nullptr)
{
	constexpr int N = 4 * LPR;
	constexpr int ROWS_PER_PASS = 256 / LPR;  // rows covered by the CTA per pass
	pdl_launch_dependents();
	pdl_wait();  // x, dt, B, C (and z) come from the kernel before this one; no-ops for a normal launch
	const int64_t bh = blockIdx.x;            // one CTA per (batch, head)
	const int h = static_cast<int>(bh % H);
	const int64_t b = bh / H;
	const int g = h / (H / G);
	const int sub = threadIdx.x % LPR;
	const int prow = threadIdx.x / LPR;
	float* sbase = state + bh * static_cast<int64_t>(P) * N;

	float4 s[RPT];
#pragma unroll
	for (int i = 0; i < RPT; ++i)
	{
		const int p = prow + i * ROWS_PER_PASS;
		if (p < P) s[i] = *(reinterpret_cast<const float4*>(sbase + static_cast<int64_t>(p) * N) + sub);
	}
	Pack<T, 4> bv, cv;
	bv.load(Bm + b * bs + static_cast<int64_t>(g) * N + sub * 4);
	cv.load(Cm + b * cs + static_cast<int64_t>(g) * N + sub * 4);
	float dtv = ldf(dt + b * dts + h);
	float xv[RPT];
#pragma unroll
	for (int i = 0; i < RPT; ++i)
	{
		const int p = prow + i * ROWS_PER_PASS;
		xv[i] = p < P ? ldf(x + b * xs + static_cast<int64_t>(h) * P + p) : 0.f;
	}
	// GATE: rows are finished by thread p (one row each, P <= 256) after the CTA barrier below
	__shared__ float y_rows[GATE ? RPT * ROWS_PER_PASS : 1];
	float zv = 0.f, nwv = 0.f;
	if (GATE && static_cast<int>(threadIdx.x) < P)
	{
		zv = ldf(z + b * zs + static_cast<int64_t>(h) * P + threadIdx.x);
		nwv = ldf(norm_w + static_cast<int64_t>(h) * P + threadIdx.x);
	}
	if (dt_bias) dtv += dt_bias[h];
	if (dt_softplus) dtv = softplus_f32(dtv);
	const float a = a_is_log ? -expf(A[h]) : A[h];
	const float dA = expf(dtv * a);
	const float dh = D ? D[h] : 0.f;
	float bf[4], cf[4];
	bv.unpack(bf);
	cv.unpack(cf);
#pragma unroll
	for (int i = 0; i < RPT; ++i)
	{
		const int p = prow + i * ROWS_PER_PASS;
		float acc = 0.f;
		if (p < P)
		{
			const float dx = dtv * xv[i];
			float4 v = s[i];
			v.x = v.x * dA + dx * bf[0];
			v.y = v.y * dA + dx * bf[1];
			v.z = v.z * dA + dx * bf[2];
			v.w = v.w * dA + dx * bf[3];
			*(reinterpret_cast<float4*>(sbase + static_cast<int64_t>(p) * N) + sub) = v;
			acc = v.x * cf[0] + v.y * cf[1] + v.z * cf[2] + v.w * cf[3];
		}
#pragma unroll
		for (int o = LPR / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
		if (p < P && sub == 0)
		{
			const float out = acc + dh * xv[i];
			if (GATE)
				y_rows[p] = out;
			else
				stf(y + b * ys + static_cast<int64_t>(h) * P + p, out);
		}
	}
	if (GATE)
	{
		__shared__ float warp_sq[8];
		__syncthreads();
		float sq = 0.f;
		if (static_cast<int>(threadIdx.x) < P)
		{
			const float out = Cvt<T>::to_f32(Cvt<T>::from_f32(y_rows[threadIdx.x]));  // y as the tensor of type T it is between the operators
			const float g = out * silu_f32(zv);
			sq = g * g;
			stf(y + b * ys + static_cast<int64_t>(h) * P + threadIdx.x, g * nwv);
		}
		sq = warp_sum(sq);
		if ((threadIdx.x & 31) == 0) warp_sq[threadIdx.x >> 5] = sq;
		__syncthreads();
		if (threadIdx.x == 0)
		{
			float t = 0.f;
#pragma unroll
			for (int i = 0; i < 8; ++i) t += warp_sq[i];
			sumsq[bh] = t;
		}
	}
}

// Any N: one thread per (b,h,p) row.
template <typename T>
__global__ void __launch_bounds__(256) ssm_update_scalar_kernel(float* __restrict__ state, const T* __restrict__ x, int64_t xs,
	const T* __restrict__ dt, int64_t dts, const float* __restrict__ A, int a_is_log, const T* __restrict__ Bm, int64_t bs,
	const T* __restrict__ Cm, int64_t cs, const float* __restrict__ D, const float* __restrict__ dt_bias, T* __restrict__ y,
	int64_t ys, int64_t nrows, int H, int P, int G, int N, int dt_softplus)
{
	const int64_t row = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
	if (row >= nrows) return;
	const int p = static_cast<int>(row % P);
	const int64_t bh = row / P;
	const int h = static_cast<int>(bh % H);
	const int64_t b = bh / H;
	const int g = h / (H / G);
	float dtv = ldf(dt + b * dts + h);
	if (dt_bias) dtv += dt_bias[h];
	if (dt_softplus) dtv = softplus_f32(dtv);
	const float a = a_is_log ? -expf(A[h]) : A[h];
	const float dA = expf(dtv * a);
	const float xv = ldf(x + b * xs + static_cast<int64_t>(h) * P + p);
	const float dx = dtv * xv;
	float acc = 0.f;
	for (int n = 0; n < N; ++n)
	{
		const float s = state[row * N + n] * dA + dx * ldf(Bm + b * bs + static_cast<int64_t>(g) * N + n);
		state[row * N + n] = s;
		acc += s * ldf(Cm + b * cs + static_cast<int64_t>(g) * N + n);
	}
	if (D) acc += D[h] * xv;
	stf(y + b * ys + static_cast<int64_t>(h) * P + p, acc);
}

template <typename T, bool GATE = false>
static int ssm_update(float* state, const void* x, int64_t xs, const void* dt, int64_t dts, const float* A, int a_is_log,
	const void* Bm, int64_t bs, const void* Cm, int64_t cs, const float* D, const float* dt_bias, void* y, int64_t ys,
	int64_t batch, int64_t H, int64_t P, int64_t G, int64_t N, int dt_softplus, cudaStream_t st, const void* z = nullptr, int64_t zs = 0,
	const void* norm_w = nullptr, float* sumsq = nullptr)
{
	const int64_t nrows = batch * H * P;
	const T* xp = static_cast<const T*>(x);
	const T* dtp = static_cast<const T*>(dt);
	const T* bp = static_cast<const T*>(Bm);
	const T* cp = static_cast<const T*>(Cm);
	T* yp = static_cast<T*>(y);
	const T* zp = static_cast<const T*>(z);
	const T* nwp = static_cast<const T*>(norm_w);
	const int h = static_cast<int>(H), p = static_cast<int>(P), g = static_cast<int>(G);
#define B200_SSM_LAUNCH(LPR)                                                                                       \
	{                                                                                                              \
		constexpr int RPP = 256 / LPR;                                                                             \
		const int64_t blocks = batch * H;                                                                          \
		if (blocks > 0x7fffffffLL) return B200_ERR_UNSUPPORTED;                                                    \
		const unsigned gb = static_cast<unsigned>(blocks);                                                         \
		if (P <= RPP)                                                                                              \
			launch_rc = launch_chained(GATE && pdl_enabled(), ssm_update_vec_kernel<T, LPR, 1, GATE>, dim3(gb), dim3(256), 0, st, state, xp, xs, \
					dtp, dts, A, a_is_log, bp, bs, cp, cs, D, dt_bias, yp, ys, h, p, g, dt_softplus, zp, zs, nwp, sumsq);                                                                     \
		else if (P <= 2 * RPP)                                                                                     \
			launch_rc = launch_chained(GATE && pdl_enabled(), ssm_update_vec_kernel<T, LPR, 2, GATE>, dim3(gb), dim3(256), 0, st, state, xp, xs, \
					dtp, dts, A, a_is_log, bp, bs, cp, cs, D, dt_bias, yp, ys, h, p, g, dt_softplus, zp, zs, nwp, sumsq);                                                                     \
		else if (P <= 4 * RPP)                                                                                     \
			launch_rc = launch_chained(GATE && pdl_enabled(), ssm_update_vec_kernel<T, LPR, 4, GATE>, dim3(gb), dim3(256), 0, st, state, xp, xs, \
					dtp, dts, A, a_is_log, bp, bs, cp, cs, D, dt_bias, yp, ys, h, p, g, dt_softplus, zp, zs, nwp, sumsq);                                                                     \
		else if (P <= 8 * RPP)                                                                                     \
			launch_rc = launch_chained(GATE && pdl_enabled(), ssm_update_vec_kernel<T, LPR, 8, GATE>, dim3(gb), dim3(256), 0, st, state, xp, xs, \
					dtp, dts, A, a_is_log, bp, bs, cp, cs, D, dt_bias, yp, ys, h, p, g, dt_softplus, zp, zs, nwp, sumsq);                                                                     \
		else                                                                                                       \
			vec_ok = false;                                                                                        \
	}
	cudaError_t launch_rc = cudaSuccess;
	// B and C are read as 4-element vectors: their rows must keep 4-element alignment
	const size_t vbytes = 4 * sizeof(T);
	bool vec_ok = aligned16(state) && (reinterpret_cast<uintptr_t>(Bm) % vbytes) == 0 && (reinterpret_cast<uintptr_t>(Cm) % vbytes) == 0 &&
		bs % 4 == 0 && cs % 4 == 0 && (N == 128 || N == 64 || N == 32 || N == 16);
	if (vec_ok && N == 128) B200_SSM_LAUNCH(32)
	else if (vec_ok && N == 64) B200_SSM_LAUNCH(16)
	else if (vec_ok && N == 32) B200_SSM_LAUNCH(8)
	else if (vec_ok && N == 16) B200_SSM_LAUNCH(4)
	if (!vec_ok)
	{
		if (GATE) return B200_ERR_UNSUPPORTED;  // callers check ssm_update_gated_applies first
		const int64_t blocks = cdiv(nrows, 256);
		if (blocks > 0x7fffffffLL) return B200_ERR_UNSUPPORTED;
		ssm_update_scalar_kernel<T><<<static_cast<unsigned>(blocks), 256, 0, st>>>(state, xp, xs, dtp, dts, A, a_is_log, bp, bs,
			cp, cs, D, dt_bias, yp, ys, nrows, h, p, g, static_cast<int>(N), dt_softplus);
	}
#undef B200_SSM_LAUNCH
	B200_CUDA_TRY(launch_rc);
	B200_LAUNCH_CHECK();
	return B200_OK;
}

// Gated form used by the fused decode step (f16): see the GATE note above. sumsq is [batch, H].
bool ssm_update_gated_applies(int64_t P, int64_t N, int64_t G)
{
	const int lpr = static_cast<int>(N / 4);
	return (N == 128 || N == 64 || N == 32 || N == 16) && P <= 8 * (256 / lpr) && (G * N) % 4 == 0;
}

int ssm_update_gated_f16(float* state, const void* x, int64_t xs, const void* dt, int64_t dts, const float* A, int a_is_log, const void* Bm,
	int64_t bs, const void* Cm, int64_t cs, const float* D, const float* dt_bias, void* y, int64_t ys, const void* z, int64_t zs,
	const void* norm_w, float* sumsq, int64_t batch, int64_t H, int64_t P, int64_t G, int64_t N, int dt_softplus, cudaStream_t st)
{
	return ssm_update<__half, true>(state, x, xs, dt, dts, A, a_is_log, Bm, bs, Cm, cs, D, dt_bias, y, ys, batch, H, P, G, N, dt_softplus, st,
		z, zs, norm_w, sumsq);
}

}  // namespace b200

using namespace b200;

extern "C" int b200_selective_state_update(int dtype, float* ssm_state, const void* x, int64_t x_stride, const void* dt,
	int64_t dt_stride, const float* A, int a_is_log, const void* B, int64_t B_stride, const void* C, int64_t C_stride,
	const float* D, const float* dt_bias, void* y, int64_t y_stride,
	int64_t batch, int64_t H, int64_t P, int64_t G, int64_t N, int dt_softplus, void* stream)
{
	if (!ssm_state || !x || !dt || !A || !B || !C || !y) return B200_ERR_NULL;
	if (batch < 0 || H <= 0 || P <= 0 || G <= 0 || N <= 0 || H % G != 0) return B200_ERR_BAD_SHAPE;
	if (x_stride < H * P || y_stride < H * P || dt_stride < H || B_stride < G * N || C_stride < G * N) return B200_ERR_BAD_SHAPE;
	if (batch == 0) return B200_OK;
	cudaStream_t st = static_cast<cudaStream_t>(stream);
	if (dtype == B200_F16)
		return ssm_update<__half>(ssm_state, x, x_stride, dt, dt_stride, A, a_is_log, B, B_stride, C, C_stride, D, dt_bias, y,
			y_stride, batch, H, P, G, N, dt_softplus, st);
	if (dtype == B200_F32)
		return ssm_update<float>(ssm_state, x, x_stride, dt, dt_stride, A, a_is_log, B, B_stride, C, C_stride, D, dt_bias, y,
			y_stride, batch, H, P, G, N, dt_softplus, st);
	return B200_ERR_UNSUPPORTED;
}
