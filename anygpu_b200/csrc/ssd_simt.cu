// SSD chunked selective scan: dt/cumsum and state-passing stages (all dtypes) and exact-fp32 SIMT versions of
// the two contraction stages. The SIMT contractions serve Tensor<float32> callers (fp32 end to end, like the
// reference's CPU path); f16 callers take the tensor-core stages in ssd_tc.cu.
#include "ssd_common.cuh"
#include "conv_dt_bodies.cuh"

namespace b200 {

// ---- stage 1: dt = softplus(dt_raw + bias); dAcs = cumsum_l(dt * A) within each chunk -------------------------
// grid (b*nchunks, ceil(H/8)), 256 threads. Positions past seqlen hold dt_raw = 0 BEFORE bias and softplus,
// exactly as the reference pads (scripts/zamba2/mamba_chunk_scan_comb.py:38-45).
template <typename T>
__global__ void __launch_bounds__(256) ssd_dt_cumsum_kernel(const T* __restrict__ dt, int64_t dts, const float* __restrict__ A,
	int a_is_log, const float* __restrict__ dt_bias, int dt_softplus, int64_t seqlen, int H, int Q, int nchunks,
	float* __restrict__ dt_out, float* __restrict__ dacs_out, float* __restrict__ colf_out)
{
	extern __shared__ float sdt[];  // [Q][kCsHeads + 1]
	ssd_dt_cumsum_body<T>(dt, dts, A, a_is_log, dt_bias, dt_softplus, seqlen, H, Q, nchunks, dt_out, dacs_out, colf_out, sdt, blockIdx.x,
		blockIdx.y);
}

template <typename T>
int ssd_dt_cumsum(const T* dt, int64_t dts, const float* A, int a_is_log, const float* dt_bias, int dt_softplus,
	const SsdDims& d, const SsdWorkspace& w, cudaStream_t st)
{
	const dim3 g(static_cast<unsigned>(d.batch * d.nchunks), static_cast<unsigned>(cdiv(d.H, kCsHeads)));
	const size_t smem = static_cast<size_t>(d.Q) * (kCsHeads + 1) * sizeof(float);
	ssd_dt_cumsum_kernel<T><<<g, 256, smem, st>>>(dt, dts, A, a_is_log, dt_bias, dt_softplus, d.seqlen, d.H, d.Q, d.nchunks,
		w.dt, w.dacs, w.colf);
	B200_LAUNCH_CHECK();
	return B200_OK;
}
template int ssd_dt_cumsum<__half>(const __half*, int64_t, const float*, int, const float*, int, const SsdDims&, const SsdWorkspace&, cudaStream_t);
template int ssd_dt_cumsum<float>(const float*, int64_t, const float*, int, const float*, int, const SsdDims&, const SsdWorkspace&, cudaStream_t);

// ---- stage 2 (SIMT): chunk states --------------------------------------------------------------------------
// grid (b*nchunks*H, ceil(P/64), ceil(N/64)), 16x16 threads, each a 4x4 patch of the [P x N] state.
template <typename T>
__global__ void __launch_bounds__(256) ssd_chunk_state_simt_kernel(const T* __restrict__ x, int64_t xs, const T* __restrict__ Bm,
	int64_t bs, const float* __restrict__ dt, const float* __restrict__ dacs, float* __restrict__ states, int64_t seqlen, int H,
	int P, int G, int N, int Q, int nchunks)
{
	__shared__ __align__(16) float sx[32][64 + 4];  // [l][p] scaled x
	__shared__ __align__(16) float sb[32][64 + 4];  // [l][n]
	const int h = blockIdx.x % H;
	const int64_t bc = blockIdx.x / H;
	const int c = static_cast<int>(bc % nchunks);
	const int64_t b = bc / nchunks;
	const int g = h / (H / G);
	const int p0 = blockIdx.y * 64, n0 = blockIdx.z * 64;
	const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
	const int64_t cbase = ((b * H + h) * nchunks + c) * static_cast<int64_t>(Q);
	const float last = dacs[cbase + Q - 1];
	float acc[4][4] = {};
	for (int l0 = 0; l0 < Q; l0 += 32)
	{
		for (int idx = threadIdx.x; idx < 32 * 64; idx += 256)
		{
			const int ll = idx >> 6, e = idx & 63;
			const int l = l0 + ll;
			const int64_t t = static_cast<int64_t>(c) * Q + l;
			float xv = 0.f, bv = 0.f;
			if (l < Q && t < seqlen)
			{
				const float sc = expf(last - dacs[cbase + l]) * dt[cbase + l];
				if (p0 + e < P) xv = ldf(x + (b * seqlen + t) * xs + static_cast<int64_t>(h) * P + p0 + e) * sc;
				if (n0 + e < N) bv = ldf(Bm + (b * seqlen + t) * bs + static_cast<int64_t>(g) * N + n0 + e);
			}
			sx[ll][e] = xv;
			sb[ll][e] = bv;
		}
		__syncthreads();
#pragma unroll 8
		for (int ll = 0; ll < 32; ++ll)
		{
			const float4 xa = *reinterpret_cast<const float4*>(&sx[ll][ty * 4]);
			const float4 ba = *reinterpret_cast<const float4*>(&sb[ll][tx * 4]);
			const float xr[4] = { xa.x, xa.y, xa.z, xa.w };
			const float br[4] = { ba.x, ba.y, ba.z, ba.w };
#pragma unroll
			for (int i = 0; i < 4; ++i)
#pragma unroll
				for (int j = 0; j < 4; ++j) acc[i][j] += xr[i] * br[j];
		}
		__syncthreads();
	}
	float* out = states + (((b * nchunks + c) * H + h) * static_cast<int64_t>(P)) * N;
#pragma unroll
	for (int i = 0; i < 4; ++i)
#pragma unroll
		for (int j = 0; j < 4; ++j)
		{
			const int p = p0 + ty * 4 + i, n = n0 + tx * 4 + j;
			if (p < P && n < N) out[static_cast<int64_t>(p) * N + n] = acc[i][j];
		}
}

template <typename T>
int ssd_chunk_state_simt(const T* x, int64_t xs, const T* Bm, int64_t bs, const SsdDims& d, const SsdWorkspace& w, cudaStream_t st)
{
	const dim3 g(static_cast<unsigned>(d.batch * d.nchunks * d.H), static_cast<unsigned>(cdiv(d.P, 64)),
		static_cast<unsigned>(cdiv(d.N, 64)));
	ssd_chunk_state_simt_kernel<T><<<g, 256, 0, st>>>(x, xs, Bm, bs, w.dt, w.dacs, w.states, d.seqlen, d.H, d.P, d.G, d.N, d.Q,
		d.nchunks);
	B200_LAUNCH_CHECK();
	return B200_OK;
}
template int ssd_chunk_state_simt<__half>(const __half*, int64_t, const __half*, int64_t, const SsdDims&, const SsdWorkspace&, cudaStream_t);
template int ssd_chunk_state_simt<float>(const float*, int64_t, const float*, int64_t, const SsdDims&, const SsdWorkspace&, cudaStream_t);

// ---- stage 3: state passing across chunks --------------------------------------------------------------------
// One thread per 4 consecutive state elements walks the chunks: states[c] <- state before chunk c, carrying the running
// state in registers. Bandwidth-bound (one read + one write of the chunk states): the loads of 8 chunks are issued
// together, ahead of the serial recurrence, so the dependent chain never waits on memory more than once per 8 chunks.
constexpr int kSpBatch = 8;

__global__ void __launch_bounds__(256) ssd_state_passing_kernel(float* __restrict__ states, __half* __restrict__ prev16,
	const float* __restrict__ dacs, const float* init, float* fin /* may alias init: every thread reads its slice first */, int H, int PN,
	int Q, int nchunks, int write_prev /* 0: only `fin` is produced, the chunk states stay as they are */)
{
	const int i = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
	if (i >= PN) return;
	const int h = blockIdx.y;
	const int64_t b = blockIdx.z;
	const int64_t cstride = static_cast<int64_t>(H) * PN;  // elements between consecutive chunks
	float* sp = states + (b * nchunks * H + h) * static_cast<int64_t>(PN) + i;
	__half* pp = prev16 ? prev16 + (b * nchunks * H + h) * static_cast<int64_t>(PN) + i : nullptr;
	const float* dl = dacs + (b * H + h) * static_cast<int64_t>(nchunks) * Q + (Q - 1);  // last dAcs of chunk c at dl[c*Q]
	float4 s = init ? *reinterpret_cast<const float4*>(init + (b * H + h) * static_cast<int64_t>(PN) + i) : make_float4(0.f, 0.f, 0.f, 0.f);
	for (int c0 = 0; c0 < nchunks; c0 += kSpBatch)
	{
		float4 cur[kSpBatch];
		float dec[kSpBatch];
#pragma unroll
		for (int j = 0; j < kSpBatch; ++j)
		{
			if (c0 + j < nchunks)
			{
				cur[j] = *reinterpret_cast<const float4*>(sp + (c0 + j) * cstride);
				dec[j] = dl[static_cast<int64_t>(c0 + j) * Q];
			}
		}
#pragma unroll
		for (int j = 0; j < kSpBatch; ++j)
		{
			if (c0 + j < nchunks)
			{
				// the state before chunk c replaces the chunk's own state: in fp32 for the SIMT scan, as f16 for the tensor-core scan
				if (write_prev && pp == nullptr) *reinterpret_cast<float4*>(sp + (c0 + j) * cstride) = s;
				if (write_prev && pp)
				{
					__half2* q = reinterpret_cast<__half2*>(pp + (c0 + j) * cstride);
					q[0] = __floats2half2_rn(s.x, s.y);
					q[1] = __floats2half2_rn(s.z, s.w);
				}
				const float d = __expf(dec[j]);
				s.x = s.x * d + cur[j].x;
				s.y = s.y * d + cur[j].y;
				s.z = s.z * d + cur[j].z;
				s.w = s.w * d + cur[j].w;
			}
		}
	}
	if (fin) *reinterpret_cast<float4*>(fin + (b * H + h) * static_cast<int64_t>(PN) + i) = s;
}

int ssd_state_passing(const float* initial_states, float* final_states, bool write_prev16, const SsdDims& d, const SsdWorkspace& w,
	cudaStream_t st, bool write_prev)
{
	const int PN = d.P * d.N;
	if (PN % 4 != 0 || (initial_states && !aligned16(initial_states)) || (final_states && !aligned16(final_states)))
		return B200_ERR_MISALIGNED;
	const dim3 g(static_cast<unsigned>(cdiv(PN / 4, 256)), static_cast<unsigned>(d.H), static_cast<unsigned>(d.batch));
	if (g.z > 65535u || g.y > 65535u) return B200_ERR_UNSUPPORTED;
	ssd_state_passing_kernel<<<g, 256, 0, st>>>(w.states, write_prev16 ? w.prev16 : nullptr, w.dacs, initial_states, final_states, d.H,
		PN, d.Q, d.nchunks, write_prev ? 1 : 0);
	B200_LAUNCH_CHECK();
	return B200_OK;
}

// Sum over the chunks of a segment of the per-chunk total of dt*A, per (batch, head): the log of the factor by which the segment
// decays a state that enters it (used when a sequence is split over GPUs).
__global__ void __launch_bounds__(256) ssd_segment_logdecay_kernel(const float* __restrict__ dacs, float* __restrict__ out, int64_t bh,
	int Q, int nchunks)
{
	const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
	if (i >= bh) return;
	const float* p = dacs + i * static_cast<int64_t>(nchunks) * Q + (Q - 1);
	float s = 0.f;
	for (int c = 0; c < nchunks; ++c) s += p[static_cast<int64_t>(c) * Q];
	out[i] = s;
}

int ssd_segment_logdecay(float* out, const SsdDims& d, const SsdWorkspace& w, cudaStream_t st)
{
	const int64_t bh = d.batch * d.H;
	ssd_segment_logdecay_kernel<<<static_cast<unsigned>(cdiv(bh, 256)), 256, 0, st>>>(w.dacs, out, bh, d.Q, d.nchunks);
	B200_LAUNCH_CHECK();
	return B200_OK;
}

// state_in = state entering segment `nseg` of a sequence split into segments: h <- exp(logdecay_q) * h + seg_state_q for
// q = 0 .. nseg-1, from the per-segment results of zero-state passes (seg_states [nseg, b*H*P*N], seg_logdecay [nseg, b*H]).
__global__ void __launch_bounds__(256) ssd_segment_prefix_kernel(const float* __restrict__ seg_states, const float* __restrict__ seg_logdecay,
	int nseg, int64_t total, int64_t bh, int PN, float* __restrict__ state_in)
{
	const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
	if (i >= total) return;
	const int64_t ibh = i / PN;
	float h = 0.f;
	for (int q = 0; q < nseg; ++q) h = h * __expf(seg_logdecay[q * bh + ibh]) + seg_states[q * total + i];
	state_in[i] = h;
}

// ---- stage 4 (SIMT): chunk scan -----------------------------------------------------------------------------
// grid (b*nchunks*H, ceil(Q/64), ceil(P/64)), 16x16 threads, each a 4x4 patch of the [64 l x 64 p] output tile.
template <typename T>
__global__ void __launch_bounds__(256) ssd_chunk_scan_simt_kernel(const T* __restrict__ x, int64_t xs, const T* __restrict__ Bm,
	int64_t bs, const T* __restrict__ Cm, int64_t cs, const float* __restrict__ D, const float* __restrict__ dt,
	const float* __restrict__ dacs, const float* __restrict__ prev, T* __restrict__ y, int64_t ys, int64_t seqlen, int H, int P,
	int G, int N, int Q, int nchunks)
{
	// s_x (x tile [s][p]) shares storage with s_a / s_b (C tile [l][n-slice]; B tile [s][n-slice] or prev tile
	// [p][n-slice]): their uses are separated by block barriers.
	__shared__ __align__(16) float s_buf[64 * (64 + 4)];
	__shared__ __align__(16) float s_s[64][64 + 4];  // decayed scores [l][s]
	float (*s_a)[33] = reinterpret_cast<float (*)[33]>(s_buf);
	float (*s_b)[33] = reinterpret_cast<float (*)[33]>(s_buf + 64 * 33);
	float (*s_x)[64 + 4] = reinterpret_cast<float (*)[64 + 4]>(s_buf);
	__shared__ float s_dl[64], s_ds[64], s_dts[64];
	const int h = blockIdx.x % H;
	const int64_t bc = blockIdx.x / H;
	const int c = static_cast<int>(bc % nchunks);
	const int64_t b = bc / nchunks;
	const int g = h / (H / G);
	const int l0 = blockIdx.y * 64, p0 = blockIdx.z * 64;
	const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
	const int64_t cbase = ((b * H + h) * nchunks + c) * static_cast<int64_t>(Q);
	const int64_t tok0 = b * seqlen + static_cast<int64_t>(c) * Q;  // first token of the chunk
	const int64_t valid = min(static_cast<int64_t>(Q), seqlen - static_cast<int64_t>(c) * Q);  // tokens of this chunk inside the sequence

	if (threadIdx.x < 64)
	{
		const int l = l0 + threadIdx.x;
		s_dl[threadIdx.x] = l < Q ? dacs[cbase + l] : 0.f;
	}

	// part 1: acc_prev[l,p] = sum_n C[l,n] prev[p,n]
	float accp[4][4] = {};
	const float* pst = prev + (((b * nchunks + c) * H + h) * static_cast<int64_t>(P)) * N;
	for (int n0 = 0; n0 < N; n0 += 32)
	{
		for (int idx = threadIdx.x; idx < 64 * 32; idx += 256)
		{
			const int r = idx >> 5, e = idx & 31;
			const int n = n0 + e;
			const int l = l0 + r, p = p0 + r;
			s_a[r][e] = (l < valid && n < N) ? ldf(Cm + (tok0 + l) * cs + static_cast<int64_t>(g) * N + n) : 0.f;
			s_b[r][e] = (p < P && n < N) ? pst[static_cast<int64_t>(p) * N + n] : 0.f;
		}
		__syncthreads();
#pragma unroll 8
		for (int e = 0; e < 32; ++e)
		{
			float ar[4], br[4];
#pragma unroll
			for (int i = 0; i < 4; ++i) { ar[i] = s_a[ty * 4 + i][e]; br[i] = s_b[tx * 4 + i][e]; }
#pragma unroll
			for (int i = 0; i < 4; ++i)
#pragma unroll
				for (int j = 0; j < 4; ++j) accp[i][j] += ar[i] * br[j];
		}
		__syncthreads();
	}

	// part 2: acc[l,p] = sum_{s<=l} (C[l].B[s]) exp(dAcs[l]-dAcs[s]) dt[s] x[s,p]
	float acc[4][4] = {};
	const int s_end = min(l0 + 64, static_cast<int>(valid));  // causal: s <= l < l0+64
	for (int s0 = 0; s0 < s_end; s0 += 64)
	{
		if (threadIdx.x < 64)
		{
			const int s = s0 + threadIdx.x;
			s_ds[threadIdx.x] = s < Q ? dacs[cbase + s] : 0.f;
			s_dts[threadIdx.x] = s < Q ? dt[cbase + s] : 0.f;
		}
		float sc[4][4] = {};
		for (int n0 = 0; n0 < N; n0 += 32)
		{
			for (int idx = threadIdx.x; idx < 64 * 32; idx += 256)
			{
				const int r = idx >> 5, e = idx & 31;
				const int n = n0 + e;
				const int l = l0 + r, s = s0 + r;
				s_a[r][e] = (l < valid && n < N) ? ldf(Cm + (tok0 + l) * cs + static_cast<int64_t>(g) * N + n) : 0.f;
				s_b[r][e] = (s < valid && n < N) ? ldf(Bm + (tok0 + s) * bs + static_cast<int64_t>(g) * N + n) : 0.f;
			}
			__syncthreads();
#pragma unroll 8
			for (int e = 0; e < 32; ++e)
			{
				float ar[4], br[4];
#pragma unroll
				for (int i = 0; i < 4; ++i) { ar[i] = s_a[ty * 4 + i][e]; br[i] = s_b[tx * 4 + i][e]; }
#pragma unroll
				for (int i = 0; i < 4; ++i)
#pragma unroll
					for (int j = 0; j < 4; ++j) sc[i][j] += ar[i] * br[j];
			}
			__syncthreads();
		}
		// decay, dt and causal mask; stage scores and the x tile
#pragma unroll
		for (int i = 0; i < 4; ++i)
#pragma unroll
			for (int j = 0; j < 4; ++j)
			{
				const int lr = ty * 4 + i, sr = tx * 4 + j;
				const int l = l0 + lr, s = s0 + sr;
				float v = 0.f;
				if (s <= l && l < valid) v = sc[i][j] * expf(s_dl[lr] - s_ds[sr]) * s_dts[sr];
				s_s[lr][sr] = v;
			}
		for (int idx = threadIdx.x; idx < 64 * 64; idx += 256)
		{
			const int r = idx >> 6, e = idx & 63;
			const int s = s0 + r, p = p0 + e;
			s_x[r][e] = (s < valid && p < P) ? ldf(x + (tok0 + s) * xs + static_cast<int64_t>(h) * P + p) : 0.f;
		}
		__syncthreads();
#pragma unroll 8
		for (int sr = 0; sr < 64; ++sr)
		{
			const float4 xa = *reinterpret_cast<const float4*>(&s_x[sr][tx * 4]);
			const float xr[4] = { xa.x, xa.y, xa.z, xa.w };
#pragma unroll
			for (int i = 0; i < 4; ++i)
			{
				const float sv = s_s[ty * 4 + i][sr];
#pragma unroll
				for (int j = 0; j < 4; ++j) acc[i][j] += sv * xr[j];
			}
		}
		__syncthreads();
	}

	const float dh = D ? D[h] : 0.f;
#pragma unroll
	for (int i = 0; i < 4; ++i)
	{
		const int lr = ty * 4 + i;
		const int l = l0 + lr;
		if (l >= valid) continue;
		const float dec = expf(s_dl[lr]);
#pragma unroll
		for (int j = 0; j < 4; ++j)
		{
			const int p = p0 + tx * 4 + j;
			if (p >= P) continue;
			float out = acc[i][j] + accp[i][j] * dec;
			if (D) out += dh * ldf(x + (tok0 + l) * xs + static_cast<int64_t>(h) * P + p);
			stf(y + (tok0 + l) * ys + static_cast<int64_t>(h) * P + p, out);
		}
	}
}

template <typename T>
int ssd_chunk_scan_simt(const T* x, int64_t xs, const T* Bm, int64_t bs, const T* Cm, int64_t cs, const float* D, T* y, int64_t ys,
	const SsdDims& d, const SsdWorkspace& w, cudaStream_t st)
{
	const dim3 g(static_cast<unsigned>(d.batch * d.nchunks * d.H), static_cast<unsigned>(cdiv(d.Q, 64)),
		static_cast<unsigned>(cdiv(d.P, 64)));
	ssd_chunk_scan_simt_kernel<T><<<g, 256, 0, st>>>(x, xs, Bm, bs, Cm, cs, D, w.dt, w.dacs, w.states, y, ys, d.seqlen, d.H, d.P,
		d.G, d.N, d.Q, d.nchunks);
	B200_LAUNCH_CHECK();
	return B200_OK;
}
template int ssd_chunk_scan_simt<__half>(const __half*, int64_t, const __half*, int64_t, const __half*, int64_t, const float*, __half*, int64_t, const SsdDims&, const SsdWorkspace&, cudaStream_t);
template int ssd_chunk_scan_simt<float>(const float*, int64_t, const float*, int64_t, const float*, int64_t, const float*, float*, int64_t, const SsdDims&, const SsdWorkspace&, cudaStream_t);

int ssd_segment_prefix(const float* seg_states, const float* seg_logdecay, int nseg, int64_t batch, int64_t H, int64_t P, int64_t N,
	float* state_in, cudaStream_t st)
{
	const int64_t total = batch * H * P * N;
	if (P * N > 0x7fffffffLL) return B200_ERR_UNSUPPORTED;
	ssd_segment_prefix_kernel<<<static_cast<unsigned>(cdiv(total, 256)), 256, 0, st>>>(seg_states, seg_logdecay, nseg, total, batch * H,
		static_cast<int>(P * N), state_in);
	B200_LAUNCH_CHECK();
	return B200_OK;
}

}  // namespace b200
