// Bodies of the token-major conv1d kernel and of the scan's dt stage as device functions: each is a kernel of its own
// (conv1d.cu, ssd_simt.cu) and both run side by side in ONE launch in the prefill mixer (conv_dt_fused.cu), where the dt stage
// (15 us of launch and ramp for a few MB) would otherwise sit between two bandwidth-bound kernels.
#pragma once

#include "common.cuh"

namespace b200 {

// The work of one thread of the token-major conv1d: V consecutive channels x TL consecutive tokens starting at (t0, c0).
// INTERIOR: the W-1 tokens before t0 and all TL tokens lie inside the sequence (all but the first and last token block): no
// per-row bounds tests, no initial state, unconditional stores.
template <typename T, int V, int W, int TL, bool INTERIOR>
__device__ __forceinline__ void conv1d_tok_thread(const T* __restrict__ xb, int64_t xs, const T* __restrict__ w, const T* __restrict__ bias,
	T* __restrict__ yb, int64_t ys, const T* __restrict__ init, T* __restrict__ fin, int seqlen, int dims, int64_t b, int c0, int t0)
{
	// rows t0-(W-1) .. t0+TL-1, all requested before the first use
	Pack<T, V> raw[TL + W - 1];
#pragma unroll
	for (int i = 0; i < TL + W - 1; ++i)
	{
		const int t = t0 - (W - 1) + i;
		if (INTERIOR || (t >= 0 && t < seqlen)) raw[i].load(xb + static_cast<int64_t>(t) * xs);
	}

	// weights of V channels x W taps are contiguous: vector loads where the row of a channel quad is 16-byte aligned
	float wt[W][V], bs[V];
	if constexpr (W == 4 && V == 4)
	{
		Pack<T, 4> wv[4], bv;
#pragma unroll
		for (int c = 0; c < 4; ++c) wv[c].load(w + static_cast<int64_t>(c0 + c) * 4);
		bv.load(bias + c0);
		bv.unpack(bs);
#pragma unroll
		for (int c = 0; c < 4; ++c)
		{
			float t4[4];
			wv[c].unpack(t4);
#pragma unroll
			for (int k = 0; k < 4; ++k) wt[k][c] = t4[k];
		}
	}
	else
	{
#pragma unroll
		for (int c = 0; c < V; ++c)
		{
			bs[c] = ldf(bias + c0 + c);
#pragma unroll
			for (int k = 0; k < W; ++k) wt[k][c] = ldf(w + static_cast<int64_t>(c0 + c) * W + k);
		}
	}

	float f[TL + W - 1][V];
#pragma unroll
	for (int i = 0; i < TL + W - 1; ++i)
	{
		const int t = t0 - (W - 1) + i;
		if (INTERIOR || t >= 0)
		{
			if (INTERIOR || t < seqlen) raw[i].unpack(f[i]);
			else
			{
#pragma unroll
				for (int c = 0; c < V; ++c) f[i][c] = 0.f;
			}
		}
		else
		{
			// before the sequence: initial conv_state [b, dims, W-1] (oldest first) or zeros
#pragma unroll
			for (int c = 0; c < V; ++c) f[i][c] = init ? ldf(init + (b * dims + c0 + c) * (W - 1) + (t + (W - 1))) : 0.f;
		}
	}

#pragma unroll
	for (int i = 0; i < TL; ++i)
	{
		if (INTERIOR || t0 + i < seqlen)
		{
			float out[V];
#pragma unroll
			for (int c = 0; c < V; ++c)
			{
				float acc = 0.f;  // taps first, bias last: the order of the reference operator
#pragma unroll
				for (int k = 0; k < W; ++k) acc += wt[k][c] * f[i + k][c];
				acc += bs[c];
				out[c] = silu_f32(acc);
			}
			Pack<T, V> o;
			o.pack(out);
			o.store(yb + static_cast<int64_t>(t0 + i) * ys);
		}
	}

	// the thread that consumed the last token holds the next conv_state: the W-1 inputs ending at token seqlen-1
	if (fin != nullptr && t0 + TL >= seqlen)
	{
		const int last = seqlen - 1 - t0;  // index of the last valid token inside this block, 0 <= last < TL
#pragma unroll
		for (int i = 0; i < TL; ++i)
		{
			if (i == last)
			{
#pragma unroll
				for (int k = 0; k < W - 1; ++k)
#pragma unroll
					for (int c = 0; c < V; ++c) stf(fin + (b * dims + c0 + c) * (W - 1) + k, f[i + 1 + k][c]);
			}
		}
	}
}

// One thread owns V consecutive channels and TL consecutive tokens of block (block_x, block_y = batch index).
template <typename T, int V, int W, int TL>
__device__ __forceinline__ void conv1d_tok_body(const T* __restrict__ x, int64_t xs, const T* __restrict__ w,
	const T* __restrict__ bias, T* __restrict__ y, int64_t ys, const T* __restrict__ init, T* __restrict__ fin,
	int seqlen, int dims, unsigned cvec /* ceil(dims / V) */, unsigned nwork /* cvec * token blocks */, unsigned block_x, unsigned block_y)
{
	const unsigned wid = block_x * blockDim.x + threadIdx.x;
	if (wid >= nwork) return;
	const unsigned tb = wid / cvec;
	const int c0 = static_cast<int>(wid - tb * cvec) * V;
	const int64_t b = block_y;
	const int t0 = static_cast<int>(tb) * TL;
	const T* xb = x + b * seqlen * xs + c0;
	T* yb = y + b * seqlen * ys + c0;
	if (t0 >= W - 1 && t0 + TL < seqlen)  // strictly inside: the block with the last token also writes the next conv_state
		conv1d_tok_thread<T, V, W, TL, true>(xb, xs, w, bias, yb, ys, init, nullptr, seqlen, dims, b, c0, t0);
	else
		conv1d_tok_thread<T, V, W, TL, false>(xb, xs, w, bias, yb, ys, init, fin, seqlen, dims, b, c0, t0);
}

// dt = softplus(dt_raw + bias); dAcs = cumsum_l(dt * A) within each chunk; colf = column factor of the rank-1 decay.
// Block (block_x = batch * nchunks + chunk, block_y = group of kCsHeads heads); sdt: [Q][kCsHeads + 1] floats of shared memory.
constexpr int kCsHeads = 8;

// Core of the dt stage for ONE chunk of Q positions and kCsHeads heads starting at h0: `dt_chunk` points at the raw dt of the chunk's
// first token (head 0), `valid` of its positions lie inside the sequence. Results of head h go to out0 + h * head_stride + l.
// Shared by the batched layout below and by the packed (variable-length) layout, so that both round identically.
template <typename T>
__device__ __forceinline__ void ssd_dt_cumsum_core(const T* __restrict__ dt_chunk, int64_t dts, const float* __restrict__ A, int a_is_log,
	const float* __restrict__ dt_bias, int dt_softplus, int valid, int H, int Q, int h0, int64_t out0, int64_t head_stride,
	float* __restrict__ dt_out, float* __restrict__ dacs_out, float* __restrict__ colf_out, float* sdt)
{
	for (int idx = threadIdx.x; idx < Q * kCsHeads; idx += blockDim.x)
	{
		const int l = idx / kCsHeads, hh = idx % kCsHeads;
		const int h = h0 + hh;
		float v = 0.f;
		if (h < H)
		{
			// positions past the end of the sequence: the reference pads dt with zeros before bias and softplus (they then decay
			// the final state); B200_DT_SOFTPLUS_EXACT gives them dt = 0, which leaves the state alone
			if (l < valid) v = ldf(dt_chunk + static_cast<int64_t>(l) * dts + h);
			if (l < valid || dt_softplus != B200_DT_SOFTPLUS_EXACT)
			{
				if (dt_bias) v += dt_bias[h];
				if (dt_softplus) v = softplus_f32(v);
			}
		}
		sdt[l * (kCsHeads + 1) + hh] = v;
	}
	__syncthreads();
	const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
	const int ep = (Q + 31) / 32;  // consecutive positions per lane (<= 8)
	for (int hh = wid; hh < kCsHeads; hh += blockDim.x / 32)
	{
		const int h = h0 + hh;
		if (h >= H) break;
		const float a = a_is_log ? -expf(A[h]) : A[h];
		float loc[8];
		float run = 0.f;
#pragma unroll
		for (int i = 0; i < 8; ++i)
		{
			const int l = lane * ep + i;
			float v = 0.f;
			// product and sum are rounded separately whatever the compiler knows about Q at the call site (a fused multiply-add
			// in one instantiation only would make the batched and the packed layout round differently)
			if (i < ep && l < Q) v = __fmul_rn(sdt[l * (kCsHeads + 1) + hh], a);
			run = __fadd_rn(run, v);
			loc[i] = run;
		}
		// exclusive prefix of lane totals
		float incl = run;
#pragma unroll
		for (int o = 1; o < 32; o <<= 1)
		{
			const float n = __shfl_up_sync(0xffffffffu, incl, o);
			if (lane >= o) incl += n;
		}
		const float excl = incl - run;
		// dAcs at the end of this lane's 64-position block (Q % 64 == 0: ep divides 64, a block is 64/ep consecutive lanes)
		const bool blocks64 = (Q % 64) == 0 && (64 % ep) == 0;
		const float blk_end = blocks64 ? __shfl_sync(0xffffffffu, excl + run, lane | (64 / ep - 1)) : 0.f;
		const int64_t base = out0 + static_cast<int64_t>(h) * head_stride;
#pragma unroll
		for (int i = 0; i < 8; ++i)
		{
			const int l = lane * ep + i;
			if (i < ep && l < Q)
			{
				const float dv = sdt[l * (kCsHeads + 1) + hh];
				dacs_out[base + l] = excl + loc[i];
				dt_out[base + l] = dv;
				if (blocks64 && colf_out) colf_out[base + l] = __expf(blk_end - (excl + loc[i])) * dv;
			}
		}
	}
}

template <typename T>
__device__ __forceinline__ void ssd_dt_cumsum_body(const T* __restrict__ dt, int64_t dts, const float* __restrict__ A,
	int a_is_log, const float* __restrict__ dt_bias, int dt_softplus, int64_t seqlen, int H, int Q, int nchunks,
	float* __restrict__ dt_out, float* __restrict__ dacs_out, float* __restrict__ colf_out, float* sdt, unsigned block_x, unsigned block_y)
{
	const int64_t b = block_x / nchunks;
	const int c = static_cast<int>(block_x % nchunks);
	const int64_t left = seqlen - static_cast<int64_t>(c) * Q;
	const int valid = static_cast<int>(left < 0 ? 0 : (left > Q ? Q : left));
	ssd_dt_cumsum_core<T>(dt + (b * seqlen + static_cast<int64_t>(c) * Q) * dts, dts, A, a_is_log, dt_bias, dt_softplus, valid, H, Q,
		static_cast<int>(block_y) * kCsHeads, (b * H * nchunks + c) * static_cast<int64_t>(Q), static_cast<int64_t>(nchunks) * Q, dt_out, dacs_out,
		colf_out, sdt);
}

}  // namespace b200
