// Prefill mixer: the token-major causal conv1d + SiLU over the xBC columns and the dt stage of the scan (softplus, in-chunk
// cumulative sums) in ONE launch. Both read only the in_proj output and neither depends on the other; alone, the dt stage is
// 15 us of launch latency and ramp for a few MB of data. Row 0 of the grid runs the dt blocks (scheduled first, so they
// finish inside the conv's run time), rows 1..batch the conv blocks.
#include "conv_dt_bodies.cuh"
#include "ssd_common.cuh"

namespace b200 {

template <typename T, int W>
__global__ void __launch_bounds__(128, 7) conv1d_tok_dt_fused_kernel(const T* __restrict__ x, int64_t xs, const T* __restrict__ w,
	const T* __restrict__ bias, T* __restrict__ y, int64_t ys, const T* __restrict__ init, T* __restrict__ fin, int seqlen, int dims,
	unsigned cvec, unsigned nwork,
	const T* __restrict__ dt, int64_t dts, const float* __restrict__ A, int a_is_log, const float* __restrict__ dt_bias, int dt_softplus,
	int H, int Q, int nchunks, float* __restrict__ dt_out, float* __restrict__ dacs_out, float* __restrict__ colf_out, unsigned dt_bx,
	unsigned dt_by)
{
	extern __shared__ float sdt[];  // [Q][kCsHeads + 1], used by the dt blocks only
	if (blockIdx.y == 0)
	{
		for (unsigned i = blockIdx.x; i < dt_bx * dt_by; i += gridDim.x)
		{
			ssd_dt_cumsum_body<T>(dt, dts, A, a_is_log, dt_bias, dt_softplus, seqlen, H, Q, nchunks, dt_out, dacs_out, colf_out, sdt, i % dt_bx,
				i / dt_bx);
			__syncthreads();  // sdt is reused by the next item
		}
		return;
	}
	// The scan that follows starts at the first tokens of every sequence at once: the conv CTAs are dealt so that those are written
	// last (token blocks from the end of the sequences to their start, the sequences taking turns) and are still in L2 then
	// (measured at batch 4 x 2048: scan 77.5 -> 74.5 us, this launch 43.7 -> 45.1 us, step -1.8 us).
	const unsigned nb = gridDim.y - 1;
	const unsigned lin = (blockIdx.y - 1) * gridDim.x + blockIdx.x;
	conv1d_tok_body<T, 4, W, 8>(x, xs, w, bias, y, ys, init, fin, seqlen, dims, cvec, nwork, gridDim.x - 1 - lin / nb, lin % nb);
}

// True when the fused launch covers this problem (otherwise the caller runs the two operators one after the other).
bool conv_dt_fused_applies(int dtype, const void* x, int64_t xs, const void* y, int64_t ys, const void* w, const void* bias, int64_t batch,
	int64_t seqlen, int64_t dims, int width)
{
	const size_t esz = dtype == B200_F16 ? 2 : 4;
	const uintptr_t amask = 4 * esz - 1;
	// the width-4 body reads the taps of a channel and the biases of a channel quad with one vector access each
	if (width == 4 && ((reinterpret_cast<uintptr_t>(w) & amask) != 0 || (reinterpret_cast<uintptr_t>(bias) & amask) != 0)) return false;
	return (dtype == B200_F16 || dtype == B200_F32) && width >= 1 && width <= 4 && (reinterpret_cast<uintptr_t>(x) & amask) == 0 &&
		(reinterpret_cast<uintptr_t>(y) & amask) == 0 && xs % 4 == 0 && ys % 4 == 0 && dims % 4 == 0 && batch > 0 && batch < 65535 &&
		seqlen > 0 && seqlen <= 0x7fffffffLL && dims <= 0x7fffffffLL && cdiv(dims, 4) * cdiv(seqlen, 8) <= 0x7fffffffLL;
}

template <typename T>
static int launch_fused(const void* x, int64_t xs, const void* w, const void* bias, void* y, int64_t ys, const void* init, void* fin,
	int64_t batch, int64_t seqlen, int64_t dims, int width, const void* dt, int64_t dts, const float* A, int a_is_log,
	const float* dt_bias, int dt_softplus, const SsdDims& d, const SsdWorkspace& sw, cudaStream_t st)
{
	const int64_t cvec = cdiv(dims, 4);
	const int64_t nwork = cvec * cdiv(seqlen, 8);
	const unsigned dt_bx = static_cast<unsigned>(d.batch * d.nchunks), dt_by = static_cast<unsigned>(cdiv(d.H, kCsHeads));
	const dim3 g(static_cast<unsigned>(cdiv(nwork, 128)), static_cast<unsigned>(batch + 1));
	const size_t smem = static_cast<size_t>(d.Q) * (kCsHeads + 1) * sizeof(float);
	const T* xp = static_cast<const T*>(x);
	const T* wp = static_cast<const T*>(w);
	const T* bp = static_cast<const T*>(bias);
	T* yp = static_cast<T*>(y);
	const T* ip = static_cast<const T*>(init);
	T* fp = static_cast<T*>(fin);
	const T* dp = static_cast<const T*>(dt);
	const int sl = static_cast<int>(seqlen), dm = static_cast<int>(dims);
	const unsigned cv = static_cast<unsigned>(cvec), nw = static_cast<unsigned>(nwork);
#define B200_FUSED(WW)                                                                                                                \
	conv1d_tok_dt_fused_kernel<T, WW><<<g, 128, smem, st>>>(xp, xs, wp, bp, yp, ys, ip, fp, sl, dm, cv, nw, dp, dts, A, a_is_log, dt_bias, \
		dt_softplus, d.H, d.Q, d.nchunks, sw.dt, sw.dacs, sw.colf, dt_bx, dt_by)
	switch (width)
	{
	case 1: B200_FUSED(1); break;
	case 2: B200_FUSED(2); break;
	case 3: B200_FUSED(3); break;
	default: B200_FUSED(4); break;
	}
#undef B200_FUSED
	B200_LAUNCH_CHECK();
	return B200_OK;
}

// conv1d over x [batch, seqlen, dims] (row stride xs) -> y, and the dt stage of the scan described by (batch, seqlen, H, P, G, N,
// chunk) into the scan workspace `ssd_workspace` (as b200_mamba_chunk_scan_combined lays it out).
int conv1d_tokens_with_scan_dt(int dtype, const void* x, int64_t xs, const void* w, const void* bias, void* y, int64_t ys,
	const void* init, void* fin, int64_t batch, int64_t seqlen, int64_t dims, int width, const void* dt, int64_t dts, const float* A,
	int a_is_log, const float* dt_bias, int dt_softplus, int64_t H, int64_t P, int64_t G, int64_t N, int64_t chunk, void* ssd_workspace,
	size_t ssd_workspace_bytes, cudaStream_t st)
{
	if (chunk <= 0 || chunk > 256) return B200_ERR_UNSUPPORTED;
	const SsdDims d{ batch, seqlen, static_cast<int>(H), static_cast<int>(P), static_cast<int>(G), static_cast<int>(N),
		static_cast<int>(chunk), static_cast<int>(cdiv(seqlen, chunk)) };
	const SsdWorkspace sw = ssd_carve(ssd_workspace, d);
	if (ssd_workspace_bytes < sw.bytes) return B200_ERR_WORKSPACE;
	if (dtype == B200_F16)
		return launch_fused<__half>(x, xs, w, bias, y, ys, init, fin, batch, seqlen, dims, width, dt, dts, A, a_is_log, dt_bias, dt_softplus, d,
			sw, st);
	return launch_fused<float>(x, xs, w, bias, y, ys, init, fin, batch, seqlen, dims, width, dt, dts, A, a_is_log, dt_bias, dt_softplus, d, sw,
		st);
}

}  // namespace b200
