// Packed variable-length batches in a fixed number of launches (f16): the token-major conv1d + SiLU and the scan's dt stage
// of ALL sequences in one launch, then the one-kernel scan over (sequence, head) pairs. The packing follows the `cu_seqlens`
// convention that scripts/zamba2/mamba_chunk_scan_comb.py:164-166 leaves unsupported: sequence s owns rows cu[s] .. cu[s+1]-1.
// Nothing crosses a boundary: the conv taps before a sequence's first token read zeros, the cumulative sums of dt*A restart
// at every 128-token block of a sequence, and a block that a sequence does not fill carries dt = 0 for the rest (the scan then
// neither reads those columns nor writes those rows). Work items are (sequence, block) pairs listed by the host in small
// index arrays, so a batch of many short sequences costs what one long sequence of the same token count costs.
#include <vector>

#include "conv_dt_bodies.cuh"
#include "ssd_common.cuh"

namespace b200 {

constexpr int kVarBlk = 128;  // tokens per scan block (the scan kernel's block size)

// dt = softplus(dt_raw + bias) and the in-block cumulative sum of dt * A for one 128-token block of one sequence and kCsHeads
// heads (the same code as the batched dt stage, so that a packed sequence rounds like the same sequence alone).
// item = block index + nblk * head group. sdt: [128][kCsHeads + 1] floats.
template <typename T>
__device__ __forceinline__ void dt_block_varlen(const T* __restrict__ dt, int64_t dts, const float* __restrict__ A, int a_is_log,
	const float* __restrict__ dt_bias, int H, const int* __restrict__ cu, const int2* __restrict__ bmap, int nblk,
	float* __restrict__ dt_out, float* __restrict__ dacs_out, float* sdt, unsigned item)
{
	const int gc = static_cast<int>(item % nblk);
	const int h0 = static_cast<int>(item / nblk) * kCsHeads;
	const int2 sc = bmap[gc];  // (sequence, block inside it)
	const int tok0 = cu[sc.x];
	const int left = cu[sc.x + 1] - tok0 - sc.y * kVarBlk;
	ssd_dt_cumsum_core<T>(dt + (static_cast<int64_t>(tok0) + sc.y * kVarBlk) * dts, dts, A, a_is_log, dt_bias, B200_DT_SOFTPLUS_EXACT,
		left > kVarBlk ? kVarBlk : left, H, kVarBlk, h0, static_cast<int64_t>(gc) * kVarBlk, static_cast<int64_t>(nblk) * kVarBlk, dt_out, dacs_out,
		nullptr, sdt);
}

// Row 0 of the grid: the dt items; row 1: the conv1d, one thread per (8-token block of a sequence, 4 channels).
template <typename T, int W>
__global__ void __launch_bounds__(128, 7) conv1d_tok_dt_varlen_kernel(const T* __restrict__ x, int64_t xs, const T* __restrict__ w,
	const T* __restrict__ bias, T* __restrict__ y, int64_t ys, T* __restrict__ fin, int dims, unsigned cvec, unsigned nwork,
	const int* __restrict__ cu, const int2* __restrict__ cmap, const T* __restrict__ dt, int64_t dts, const float* __restrict__ A, int a_is_log,
	const float* __restrict__ dt_bias, int H, const int2* __restrict__ bmap, int nblk, float* __restrict__ dt_out, float* __restrict__ dacs_out,
	unsigned dt_items)
{
	__shared__ float sdt[kVarBlk * (kCsHeads + 1)];
	if (blockIdx.y == 0)
	{
		for (unsigned i = blockIdx.x; i < dt_items; i += gridDim.x)
		{
			dt_block_varlen<T>(dt, dts, A, a_is_log, dt_bias, H, cu, bmap, nblk, dt_out, dacs_out, sdt, i);
			__syncthreads();  // sdt is reused by the next item
		}
		return;
	}
	const unsigned wid = blockIdx.x * blockDim.x + threadIdx.x;
	if (wid >= nwork) return;
	const unsigned cb = wid / cvec;
	const int c0 = static_cast<int>(wid - cb * cvec) * 4;
	const int2 sb = cmap[cb];  // (sequence, 8-token block inside it)
	const int tok0 = cu[sb.x];
	const int len = cu[sb.x + 1] - tok0;
	const int t0 = sb.y * 8;
	const T* xb = x + static_cast<int64_t>(tok0) * xs + c0;
	T* yb = y + static_cast<int64_t>(tok0) * ys + c0;
	if (t0 >= W - 1 && t0 + 8 < len)  // strictly inside: the block with the last token also writes the sequence's conv_state
		conv1d_tok_thread<T, 4, W, 8, true>(xb, xs, w, bias, yb, ys, nullptr, nullptr, len, dims, sb.x, c0, t0);
	else
		conv1d_tok_thread<T, 4, W, 8, false>(xb, xs, w, bias, yb, ys, nullptr, fin, len, dims, sb.x, c0, t0);
}

// True when the packed path covers the problem (f16, vector-aligned xBC slice, the shapes of the one-kernel scan).
bool mixer_varlen_fused_applies(int dtype, const void* xbc_in, int64_t xs, const void* xbc, int64_t conv_dim, const void* conv_w,
	const void* conv_b, int width, int64_t total_tokens, int64_t nseq, int64_t H, int64_t P, int64_t G, int64_t N, const void* y, int64_t ys,
	const float* init, const float* fin)
{
	if (dtype != B200_F16 || width < 1 || width > 4 || total_tokens <= 0 || nseq <= 0) return false;
	const uintptr_t amask = 7;  // 4 f16
	if ((reinterpret_cast<uintptr_t>(xbc_in) & amask) || (reinterpret_cast<uintptr_t>(xbc) & amask) || xs % 4 || conv_dim % 4) return false;
	if (width == 4 && ((reinterpret_cast<uintptr_t>(conv_w) & amask) || (reinterpret_cast<uintptr_t>(conv_b) & amask))) return false;
	const int64_t d_inner = H * P, GN = G * N;
	const char* xo = static_cast<const char*>(xbc);
	return ssd_fused_varlen_supported(total_tokens, nseq, static_cast<int>(H), static_cast<int>(P), static_cast<int>(G), static_cast<int>(N),
		xo, conv_dim, xo + d_inner * 2, conv_dim, xo + (d_inner + GN) * 2, conv_dim, y, ys, init, fin);
}

// conv1d + SiLU over the xBC columns of all sequences, the dt stage, and the scan, for a packed f16 batch. `scratch` receives the
// index arrays and the dt stage's rows; returns B200_ERR_WORKSPACE when it is too small (the caller then runs sequence by
// sequence). cu_host: nseq + 1 non-decreasing offsets starting at 0.
int mixer_conv_ssd_varlen_f16(const void* xbc_in, int64_t xs, const void* conv_w, const void* conv_b, int width, void* xbc, int64_t conv_dim,
	void* conv_state_out, const void* dt, int64_t dts, const float* A_log, const float* dt_bias, const float* D, const float* init, void* y,
	int64_t ys, float* fin, const int64_t* cu_host, int64_t nseq, int64_t H, int64_t P, int64_t G, int64_t N, void* scratch,
	size_t scratch_bytes, cudaStream_t st)
{
	const int64_t T = cu_host[nseq];
	// host-side index arrays
	std::vector<int> cu(static_cast<size_t>(nseq) + 1), coff(static_cast<size_t>(nseq) + 1);
	std::vector<int2> bmap, cmap;
	int nblk = 0;
	for (int64_t s = 0; s < nseq; ++s)
	{
		const int len = static_cast<int>(cu_host[s + 1] - cu_host[s]);
		cu[s] = static_cast<int>(cu_host[s]);
		coff[s] = nblk;
		for (int c = 0; c < (len + kVarBlk - 1) / kVarBlk; ++c) bmap.push_back(make_int2(static_cast<int>(s), c));
		for (int c = 0; c < (len + 7) / 8; ++c) cmap.push_back(make_int2(static_cast<int>(s), c));
		nblk += (len + kVarBlk - 1) / kVarBlk;
	}
	cu[nseq] = static_cast<int>(T);
	coff[nseq] = nblk;
	// scratch layout: dt rows | dA rows ([H][nblk][128] fp32 each) | cu | coff | bmap | cmap
	const size_t rows = align_up(static_cast<size_t>(H) * nblk * kVarBlk * sizeof(float), 256);
	const size_t o_cu = 2 * rows;
	const size_t o_coff = o_cu + align_up(cu.size() * sizeof(int), 256);
	const size_t o_bmap = o_coff + align_up(coff.size() * sizeof(int), 256);
	const size_t o_cmap = o_bmap + align_up(bmap.size() * sizeof(int2), 256);
	const size_t need = o_cmap + align_up(cmap.size() * sizeof(int2), 256);
	if (need > scratch_bytes) return B200_ERR_WORKSPACE;
	char* sp = static_cast<char*>(scratch);
	float* dt_rows = reinterpret_cast<float*>(sp);
	float* dacs_rows = reinterpret_cast<float*>(sp + rows);
	int* d_cu = reinterpret_cast<int*>(sp + o_cu);
	int* d_coff = reinterpret_cast<int*>(sp + o_coff);
	int2* d_bmap = reinterpret_cast<int2*>(sp + o_bmap);
	int2* d_cmap = reinterpret_cast<int2*>(sp + o_cmap);
	// the arrays are pageable host memory: each copy is staged before the call returns, so the vectors may go out of scope
	B200_CUDA_TRY(cudaMemcpyAsync(d_cu, cu.data(), cu.size() * sizeof(int), cudaMemcpyHostToDevice, st));
	B200_CUDA_TRY(cudaMemcpyAsync(d_coff, coff.data(), coff.size() * sizeof(int), cudaMemcpyHostToDevice, st));
	if (!bmap.empty()) B200_CUDA_TRY(cudaMemcpyAsync(d_bmap, bmap.data(), bmap.size() * sizeof(int2), cudaMemcpyHostToDevice, st));
	if (!cmap.empty()) B200_CUDA_TRY(cudaMemcpyAsync(d_cmap, cmap.data(), cmap.size() * sizeof(int2), cudaMemcpyHostToDevice, st));

	const int64_t cvec = conv_dim / 4;
	const int64_t nwork = cvec * static_cast<int64_t>(cmap.size());
	const int64_t dt_items = static_cast<int64_t>(nblk) * cdiv(H, kCsHeads);
	if (nwork > 0x7fffffffLL || dt_items > 0x7fffffffLL) return B200_ERR_UNSUPPORTED;
	if (nwork > 0)
	{
		const dim3 g(static_cast<unsigned>(cdiv(nwork, 128)), 2);
		const __half* xp = static_cast<const __half*>(xbc_in);
		const __half* wp = static_cast<const __half*>(conv_w);
		const __half* bp = static_cast<const __half*>(conv_b);
		__half* yp = static_cast<__half*>(xbc);
		__half* fp = static_cast<__half*>(conv_state_out);
		const __half* dp = static_cast<const __half*>(dt);
		const int dm = static_cast<int>(conv_dim);
		const unsigned cv = static_cast<unsigned>(cvec), nw = static_cast<unsigned>(nwork), di = static_cast<unsigned>(dt_items);
#define B200_VARLEN(WW)                                                                                                                \
	conv1d_tok_dt_varlen_kernel<__half, WW><<<g, 128, 0, st>>>(xp, xs, wp, bp, yp, conv_dim, fp, dm, cv, nw, d_cu, d_cmap, dp, dts, A_log, 1, \
		dt_bias, static_cast<int>(H), d_bmap, nblk, dt_rows, dacs_rows, di)
		switch (width)
		{
		case 1: B200_VARLEN(1); break;
		case 2: B200_VARLEN(2); break;
		case 3: B200_VARLEN(3); break;
		default: B200_VARLEN(4); break;
		}
#undef B200_VARLEN
		B200_LAUNCH_CHECK();
	}
	const int64_t d_inner = H * P, GN = G * N;
	const __half* xo = static_cast<const __half*>(xbc);
	return ssd_fused_varlen_tc(xo, conv_dim, xo + d_inner, conv_dim, xo + d_inner + GN, conv_dim, D, init, static_cast<__half*>(y), ys, fin, T,
		nseq, static_cast<int>(H), static_cast<int>(G), dt_rows, dacs_rows, d_cu, d_coff, nblk, st);
}

}  // namespace b200
