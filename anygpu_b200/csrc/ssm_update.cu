// Single-token ssm_state recurrence for decode:
//   dt = softplus(dt_raw + dt_bias); h <- exp(dt*A) h + dt x (x) B; y = h.C + D x    per (batch, head).
// HBM-bound: the fp32 state [b,H,P,N] is read once and written once with 128-bit accesses (a 64-wide state row is
// 16 lanes x float4); everything else is noise next to it. The y reduction over N runs in warp shuffles.
#include "common.cuh"

namespace b200 {

// LPR lanes share one (b,h,p) row of N = 4*LPR states (LPR a power of two, 4..32). A CTA of 128 threads owns one (batch,
// head): grid (H, batch). A thread owns RPT rows, 128/LPR rows apart, and issues all of their 128-bit state loads before the
// first use, so that enough bytes are in flight per SM to cover HBM latency. B and C are read as one 8-byte (f16) or 16-byte
// (f32) vector per thread.
//
// The kernel issues ~100 instructions per 128-bit state access if written naively and is then bound by instruction issue,
// not HBM, so the per-row work is kept minimal: no integer division (2-D grid), and the y reduction of four rows over the
// LPR lanes of a group is one butterfly in which the first two steps exchange rows instead of adding all four (5-6 shuffles
// per four rows instead of 16-20); afterwards lane `sub` holds the total of row sub / (LPR/4) of each quad of rows.
//
// GATE: the output is additionally gated and weighted for the RMSNorm that follows, y <- round_T(y) * silu(z) * norm_w, and
// every warp's sum of (round_T(y) * silu(z))^2 goes to sumsq[b, h, warp] (kSsmWarps per CTA); the consumer of y applies
// rsqrt(mean + eps) (a row scale commutes with the projection that follows the norm). Nothing waits for another warp.
constexpr int kSsmThreads = 128, kSsmWarps = kSsmThreads / 32;

// 128-bit state load that the compiler keeps where it is written: all of a thread's state loads are issued back to back
// before anything else, which is what keeps enough bytes in flight (left to itself the compiler interleaves them with their
// uses in some instantiations and the kernel loses a quarter of its bandwidth).
__device__ __forceinline__ float4 ld_state(const float4* p)
{
	float4 v;
	asm volatile("ld.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
	return v;
}

template <int LPR>
__device__ __forceinline__ float quad_row_reduce(float a0, float a1, float a2, float a3, int sub)
{
	const bool hi1 = (sub & (LPR / 2)) != 0;
	float k0 = hi1 ? a2 : a0, k1 = hi1 ? a3 : a1;
	k0 += __shfl_xor_sync(0xffffffffu, hi1 ? a0 : a2, LPR / 2);
	k1 += __shfl_xor_sync(0xffffffffu, hi1 ? a1 : a3, LPR / 2);
	const bool hi0 = (sub & (LPR / 4)) != 0;
	float k = hi0 ? k1 : k0;
	k += __shfl_xor_sync(0xffffffffu, hi0 ? k0 : k1, LPR / 4);
#pragma unroll
	for (int o = LPR / 8; o > 0; o >>= 1) k += __shfl_xor_sync(0xffffffffu, k, o);
	return k;  // total of row 2*hi1 + hi0 = sub / (LPR/4)
}

template <typename T, int LPR, int RPT, bool GATE = false>
__global__ void __launch_bounds__(kSsmThreads) ssm_update_vec_kernel(float* __restrict__ state, const T* __restrict__ x, int64_t xs,
	const T* __restrict__ dt, int64_t dts, const float* __restrict__ A, int a_is_log, const T* __restrict__ Bm, int64_t bs,
	const T* __restrict__ Cm, int64_t cs, const float* __restrict__ D, const float* __restrict__ dt_bias, T* __restrict__ y,
	int64_t ys, int batch, int P, int hpg, int dt_softplus, const T* __restrict__ z = nullptr, int64_t zs = 0,
	const T* __restrict__ norm_w = nullptr, float* __restrict__ sumsq = nullptr)
{
	constexpr int N = 4 * LPR;
	constexpr int RPP = kSsmThreads / LPR;   // rows covered by the CTA per pass
	constexpr int QUADS = RPT >= 4 ? RPT / 4 : 1;  // row totals a lane ends up with
	pdl_launch_dependents();
	pdl_wait();  // x, dt, B, C (and z) come from the kernel before this one; no-ops for a normal launch
	const int h = blockIdx.x, H = gridDim.x;
	const int b = blockIdx.y + blockIdx.z * gridDim.y;
	if (b >= batch) return;
	const int g = hpg == H ? 0 : h / hpg;
	const int sub = threadIdx.x % LPR;
	const int prow = threadIdx.x / LPR;
	const int64_t bh = static_cast<int64_t>(b) * H + h;
	float4* srow = reinterpret_cast<float4*>(state + bh * static_cast<int64_t>(P) * N) + prow * LPR + sub;  // row i: + i * RPP * LPR
	const T* xrow = x + b * xs + h * P + prow;                                                            // row i: + i * RPP

	float4 s[RPT];
	bool live[RPT];
#pragma unroll
	for (int i = 0; i < RPT; ++i)
	{
		live[i] = prow + i * RPP < P;
		s[i] = ld_state(live[i] ? srow + i * RPP * LPR : srow - prow * LPR);  // dead rows read row 0 and are ignored
	}
	Pack<T, 4> bv, cv;
	bv.load(Bm + b * bs + g * N + sub * 4);
	cv.load(Cm + b * cs + g * N + sub * 4);
	float dtv = ldf(dt + b * dts + h);
	float xv[RPT];
#pragma unroll
	for (int i = 0; i < RPT; ++i) xv[i] = live[i] ? ldf(xrow + i * RPP) : 0.f;
	// rows whose totals this lane ends up with: RPT >= 4: row 4q + sub / (LPR/4) of every quad q, on lanes with sub % (LPR/4) == 0;
	// RPT < 4: row `sub` (all lanes of the group hold every total after a plain all-reduce)
	const bool owner = RPT >= 4 ? (sub % (LPR / 4)) == 0 : sub < RPT;
	const int own0 = RPT >= 4 ? sub / (LPR / 4) : sub;
	float zv[QUADS], nwv[QUADS];
	if (GATE)
	{
#pragma unroll
		for (int q = 0; q < QUADS; ++q)
		{
			const int p = prow + (4 * q + own0) * RPP;
			const bool mine = owner && p < P;
			zv[q] = mine ? ldf(z + b * zs + h * P + p) : 0.f;
			nwv[q] = mine ? ldf(norm_w + h * P + p) : 0.f;
		}
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
	for (int j = 0; j < 4; ++j) bf[j] *= dtv;  // dt * B, shared by all rows
	float acc[RPT];
#pragma unroll
	for (int i = 0; i < RPT; ++i)
	{
		acc[i] = 0.f;
		if (live[i])
		{
			float4 v = s[i];
			v.x = v.x * dA + xv[i] * bf[0];
			v.y = v.y * dA + xv[i] * bf[1];
			v.z = v.z * dA + xv[i] * bf[2];
			v.w = v.w * dA + xv[i] * bf[3];
			srow[i * RPP * LPR] = v;
			acc[i] = v.x * cf[0] + v.y * cf[1] + v.z * cf[2] + v.w * cf[3];
		}
	}
	float own[QUADS], own_x[QUADS];
	if (RPT >= 4)
	{
#pragma unroll
		for (int q = 0; q < QUADS; ++q)
		{
			own[q] = quad_row_reduce<LPR>(acc[4 * q], acc[4 * q + 1], acc[4 * q + 2], acc[4 * q + 3], sub);
			const float x01 = (own0 & 1) ? xv[4 * q + 1] : xv[4 * q], x23 = (own0 & 1) ? xv[4 * q + 3] : xv[4 * q + 2];
			own_x[q] = (own0 & 2) ? x23 : x01;
		}
	}
	else
	{
		own[0] = 0.f;
		own_x[0] = 0.f;
#pragma unroll
		for (int i = 0; i < RPT; ++i)
		{
			float t = acc[i];
#pragma unroll
			for (int o = LPR / 2; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
			if (sub == i)
			{
				own[0] = t;
				own_x[0] = xv[i];
			}
		}
	}
	float sq = 0.f;
#pragma unroll
	for (int q = 0; q < QUADS; ++q)
	{
		const int p = prow + (4 * q + own0) * RPP;
		if (owner && p < P)
		{
			float out = own[q] + dh * own_x[q];
			if (GATE)
			{
				out = Cvt<T>::to_f32(Cvt<T>::from_f32(out));  // y as the tensor of type T it is between the two operators
				const float gt = out * silu_f32(zv[q]);
				sq += gt * gt;
				out = gt * nwv[q];
			}
			stf(y + b * ys + h * P + p, out);
		}
	}
	if (GATE)
	{
		sq = warp_sum(sq);
		if ((threadIdx.x & 31) == 0) sumsq[bh * kSsmWarps + (threadIdx.x >> 5)] = sq;
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
	const int p = static_cast<int>(P), hpg = static_cast<int>(H / G), nb = static_cast<int>(batch);
	// grid (H, batch) with the batch folded into y and z
	const unsigned gy = static_cast<unsigned>(batch < 32768 ? batch : 32768), gz = static_cast<unsigned>(cdiv(batch, gy));
	const dim3 grid(static_cast<unsigned>(H), gy, gz);
	cudaError_t launch_rc = cudaSuccess;
// normal launches (also inside the fused decode step: with this kernel's CTAs resident early the step measured slower)
#define B200_SSM_RPT(LPR, R)                                                                                                     \
	launch_rc = launch_chained(false, ssm_update_vec_kernel<T, LPR, R, GATE>, grid, dim3(kSsmThreads), 0, st, state, xp, \
		xs, dtp, dts, A, a_is_log, bp, bs, cp, cs, D, dt_bias, yp, ys, nb, p, hpg, dt_softplus, zp, zs, nwp, sumsq)
#define B200_SSM_LAUNCH(LPR)                                   \
	{                                                          \
		constexpr int RPP = kSsmThreads / LPR;                 \
		if (P <= RPP) B200_SSM_RPT(LPR, 1);                    \
		else if (P <= 2 * RPP) B200_SSM_RPT(LPR, 2);           \
		else if (P <= 4 * RPP) B200_SSM_RPT(LPR, 4);           \
		else if (P <= 8 * RPP) B200_SSM_RPT(LPR, 8);           \
		else if (P <= 16 * RPP) B200_SSM_RPT(LPR, 16);         \
		else vec_ok = false;                                   \
	}
	// B and C are read as 4-element vectors: their rows must keep 4-element alignment; 32-bit offsets inside one batch row
	const size_t vbytes = 4 * sizeof(T);
	bool vec_ok = aligned16(state) && (reinterpret_cast<uintptr_t>(Bm) % vbytes) == 0 && (reinterpret_cast<uintptr_t>(Cm) % vbytes) == 0 &&
		bs % 4 == 0 && cs % 4 == 0 && (N == 128 || N == 64 || N == 32 || N == 16) && H <= 65535 && H * P < (1LL << 30) && gz <= 65535;
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
			cp, cs, D, dt_bias, yp, ys, nrows, static_cast<int>(H), p, static_cast<int>(G), static_cast<int>(N), dt_softplus);
		count_launch();  // launch_chained has counted the vector kernel
	}
#undef B200_SSM_LAUNCH
#undef B200_SSM_RPT
	B200_CUDA_TRY(launch_rc);
	B200_CUDA_TRY(cudaGetLastError());
	return B200_OK;
}

// Gated form used by the fused decode step (f16): see the GATE note above. sumsq is [batch, H, ssm_update_gated_partials()].
int ssm_update_gated_partials() { return kSsmWarps; }

bool ssm_update_gated_applies(int64_t H, int64_t P, int64_t N, int64_t G)
{
	const int lpr = static_cast<int>(N / 4);
	return (N == 128 || N == 64 || N == 32 || N == 16) && P <= 16 * (kSsmThreads / lpr) && (G * N) % 4 == 0 && H <= 65535 &&
		H * P < (1LL << 30);
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
