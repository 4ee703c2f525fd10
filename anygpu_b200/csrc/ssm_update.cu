// Single-token ssm_state recurrence for decode:
//   dt = softplus(dt_raw + dt_bias); h <- exp(dt*A) h + dt x (x) B; y = h.C + D x    per (batch, head).
// HBM-bound: the fp32 state [b,H,P,N] is read once and written once with 128-bit accesses (a 64-wide state row is
// 16 lanes x float4); everything else is noise next to it. The y reduction over N runs in warp shuffles.
#include "common.cuh"

namespace b200 {

// LPR lanes share one (b,h,p) row of N = 4*LPR states. LPR is a power of two <= 32.
template <typename T, int LPR>
__global__ void __launch_bounds__(256) ssm_update_vec_kernel(float* __restrict__ state, const T* __restrict__ x, int64_t xs,
	const T* __restrict__ dt, int64_t dts, const float* __restrict__ A, int a_is_log, const T* __restrict__ Bm, int64_t bs,
	const T* __restrict__ Cm, int64_t cs, const float* __restrict__ D, const float* __restrict__ dt_bias, T* __restrict__ y,
	int64_t ys, int64_t nrows /* b*H*P */, int H, int P, int G, int dt_softplus)
{
	constexpr int N = 4 * LPR;
	const int64_t gt = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
	const int64_t row = gt / LPR;
	const int sub = static_cast<int>(gt % LPR);
	const bool active = row < nrows;
	float acc = 0.f;
	int64_t b = 0;
	int h = 0, p = 0;
	float xv = 0.f;
	if (active)
	{
		p = static_cast<int>(row % P);
		const int64_t bh = row / P;
		h = static_cast<int>(bh % H);
		b = bh / H;
		const int g = h / (H / G);
		float dtv = ldf(dt + b * dts + h);
		if (dt_bias) dtv += dt_bias[h];
		if (dt_softplus) dtv = softplus_f32(dtv);
		const float a = a_is_log ? -expf(A[h]) : A[h];
		const float dA = expf(dtv * a);
		xv = ldf(x + b * xs + static_cast<int64_t>(h) * P + p);
		const float dx = dtv * xv;
		float4* sp = reinterpret_cast<float4*>(state + row * N) + sub;
		float4 s = *sp;
		const T* bp = Bm + b * bs + static_cast<int64_t>(g) * N + sub * 4;
		const T* cp = Cm + b * cs + static_cast<int64_t>(g) * N + sub * 4;
		const float b0 = ldf(bp), b1 = ldf(bp + 1), b2 = ldf(bp + 2), b3 = ldf(bp + 3);
		const float c0 = ldf(cp), c1 = ldf(cp + 1), c2 = ldf(cp + 2), c3 = ldf(cp + 3);
		s.x = s.x * dA + dx * b0;
		s.y = s.y * dA + dx * b1;
		s.z = s.z * dA + dx * b2;
		s.w = s.w * dA + dx * b3;
		*sp = s;
		acc = s.x * c0 + s.y * c1 + s.z * c2 + s.w * c3;
	}
#pragma unroll
	for (int o = LPR / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
	if (active && sub == 0)
	{
		if (D) acc += D[h] * xv;
		stf(y + b * ys + static_cast<int64_t>(h) * P + p, acc);
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

template <typename T>
static int ssm_update(float* state, const void* x, int64_t xs, const void* dt, int64_t dts, const float* A, int a_is_log,
	const void* Bm, int64_t bs, const void* Cm, int64_t cs, const float* D, const float* dt_bias, void* y, int64_t ys,
	int64_t batch, int64_t H, int64_t P, int64_t G, int64_t N, int dt_softplus, cudaStream_t st)
{
	const int64_t nrows = batch * H * P;
	const T* xp = static_cast<const T*>(x);
	const T* dtp = static_cast<const T*>(dt);
	const T* bp = static_cast<const T*>(Bm);
	const T* cp = static_cast<const T*>(Cm);
	T* yp = static_cast<T*>(y);
	const int h = static_cast<int>(H), p = static_cast<int>(P), g = static_cast<int>(G);
#define B200_SSM_LAUNCH(LPR)                                                                                       \
	{                                                                                                              \
		const int64_t blocks = cdiv(nrows * LPR, 256);                                                             \
		if (blocks > 0x7fffffffLL) return B200_ERR_UNSUPPORTED;                                                    \
		ssm_update_vec_kernel<T, LPR><<<static_cast<unsigned>(blocks), 256, 0, st>>>(state, xp, xs, dtp, dts, A,   \
			a_is_log, bp, bs, cp, cs, D, dt_bias, yp, ys, nrows, h, p, g, dt_softplus);                            \
	}
	if (aligned16(state) && N == 128) B200_SSM_LAUNCH(32)
	else if (aligned16(state) && N == 64) B200_SSM_LAUNCH(16)
	else if (aligned16(state) && N == 32) B200_SSM_LAUNCH(8)
	else if (aligned16(state) && N == 16) B200_SSM_LAUNCH(4)
	else
	{
		const int64_t blocks = cdiv(nrows, 256);
		if (blocks > 0x7fffffffLL) return B200_ERR_UNSUPPORTED;
		ssm_update_scalar_kernel<T><<<static_cast<unsigned>(blocks), 256, 0, st>>>(state, xp, xs, dtp, dts, A, a_is_log, bp, bs,
			cp, cs, D, dt_bias, yp, ys, nrows, h, p, g, static_cast<int>(N), dt_softplus);
	}
#undef B200_SSM_LAUNCH
	B200_LAUNCH_CHECK();
	return B200_OK;
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
