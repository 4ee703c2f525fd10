// Decode projections: Y[M,N] = X[M,K] . W with M <= 128 tokens against a large weight. The job is to stream W from HBM once.
//
// There are only ceil(N/256) output tiles, far fewer than SMs, so the (tile, K-block) units are dealt out evenly to one
// CTA per SM ("stream-K"): CTA c owns the contiguous unit range [c*U/G, (c+1)*U/G), which may end one tile and begin the
// next. Each tile segment is accumulated by tcgen05.mma into one of two TMEM accumulators and written as an fp32 partial
// tile to slice `c - first_cta(tile)` of a [tile][slice][M][256] buffer; the consumer kernels add the slices of a tile in
// slice order, so the result does not depend on scheduling, and fuse the step that follows the projection:
//   in_proj  -> rounding to f16, rolling conv1d state update + SiLU for the xBC columns
//   out_proj -> the RMSNorm row scale (sum of squares collected by the recurrence kernel), rounding to f16
// The partial tiles are written and read within microseconds and stay in L2.
//
// Roles per CTA as in the prefill GEMM: warp 0 TMA producer, warp 1 MMA issuer, warps 2-5 epilogue (fp32 sub-tiles staged in
// shared memory, 128B-swizzled, and written with TMA stores as full 128-byte lines); every wait is bounded. The producer
// issues its first ring of loads before the CTA-wide setup barrier, and the weight loads before griddepcontrol.wait: the
// kernels of a decode step are launched with programmatic stream serialization, so a CTA may start while the kernel before
// it drains, and only accesses to that kernel's outputs have to wait for it.
#include "tcgen05.cuh"

namespace b200 {

namespace dgemm {
constexpr int BM = 128, BN = 256, BK = 64, THREADS = 192, RING_WARPS = 4;
constexpr int B_BYTES = BN * BK * 2;
constexpr uint32_t TMEM_COLS = 2 * BN;
constexpr int STG_BYTES = 32 * 128;  // per-warp staging tile: 32 rows x 32 fp32
template <int A_ROWS> struct Ring
{
	static constexpr int A_BYTES = A_ROWS * BK * 2;
	static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
	static constexpr int STAGES = A_ROWS == 64 ? 5 : 4;  // 200 KiB / 192 KiB of ring
	static constexpr int STG_WARPS = A_ROWS / 32;        // epilogue warps that own rows < A_ROWS
	static constexpr int STG_TOTAL = STG_WARPS * 2 * STG_BYTES;
	static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + STG_TOTAL + 1024;  // + slack to align the ring to 1024 B
};

// CTA that owns unit u when U units are dealt to G CTAs as [c*U/G, (c+1)*U/G).
__host__ __device__ inline int cta_of_unit(int64_t u, int64_t G, int64_t U) { return static_cast<int>(((u + 1) * G + U - 1) / U - 1); }
}  // namespace dgemm

// A_ROWS = 64: only 64 rows of X are fetched per stage; the MMA (M = 128) reads the following 8 KiB of the ring as rows
// 64..127 and the accumulator rows it makes of them are never stored.
template <int B_MN, int A_ROWS>
__global__ void __launch_bounds__(dgemm::THREADS, 1) gemm_f16_streamk_kernel(const __grid_constant__ CUtensorMap tmA,
	const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmP, int M, int k_blocks, int total_units, int max_seg,
	uint32_t* err_word)
{
	using namespace dgemm;
	using namespace tc;
	using R = Ring<A_ROWS>;
	constexpr int STAGES = R::STAGES, STAGE_BYTES = R::STAGE_BYTES, A_BYTES = R::A_BYTES;
	extern __shared__ uint8_t smem_raw[];
	__shared__ uint64_t bar_full[STAGES], bar_empty[STAGES], bar_tfull[2], bar_tempty[2];
	__shared__ uint32_t tmem_slot;
	__shared__ int abort_flag;

	pdl_launch_dependents();
	const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
	const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
	const int u_begin = static_cast<int>(static_cast<int64_t>(blockIdx.x) * total_units / gridDim.x);
	const int u_end = static_cast<int>(static_cast<int64_t>(blockIdx.x + 1) * total_units / gridDim.x);
	volatile int* abortp = &abort_flag;

	// one unit = one ring stage: W tile first (it never depends on the kernel before this one), then X after `dep_wait`
	auto load_unit = [&](int u, int stage, bool dep_wait) {
		const int tile = u / k_blocks;
		const int kb = u - tile * k_blocks;
		const int n0 = tile * BN;
		const uint32_t full = smem_u32(&bar_full[stage]);
		const uint32_t a_s = ring + stage * STAGE_BYTES;
		const uint32_t b_s = a_s + A_BYTES;
		mbar_arrive_expect_tx(full, STAGE_BYTES);
		if (B_MN == 0)
		{
			tma_load_2d(b_s, &tmB, full, kb * BK, n0);  // W^T [N,K]: one [256 n x 64 k] box
		}
		else
		{
#pragma unroll
			for (int j = 0; j < BN / 64; ++j)  // W [K,N]: four boxes of [64 k x 64 n] side by side, 512 B of every W row
				tma_load_2d(b_s + j * (BK * 128), &tmB, full, n0 + j * 64, kb * BK);
		}
		if (!dep_wait) tma_load_2d(a_s, &tmA, full, kb * BK, 0);
	};
	const int n_first = min(STAGES, u_end - u_begin);  // units whose loads go out before the setup barrier

	if (threadIdx.x == 0)
	{
		abort_flag = 0;
		for (int s = 0; s < STAGES; ++s)
		{
			mbar_init(smem_u32(&bar_full[s]), 1);
			mbar_init(smem_u32(&bar_empty[s]), 1);
		}
		for (int a = 0; a < 2; ++a)
		{
			mbar_init(smem_u32(&bar_tfull[a]), 1);
			mbar_init(smem_u32(&bar_tempty[a]), RING_WARPS);
		}
		fence_mbar_init();
		prefetch_tmap(&tmA);
		prefetch_tmap(&tmB);
		for (int i = 0; i < n_first; ++i) load_unit(u_begin + i, i, true);
		pdl_wait();  // X is the output of the kernel before this one
		for (int i = 0; i < n_first; ++i)
		{
			const int u = u_begin + i;
			tma_load_2d(ring + i * STAGE_BYTES, &tmA, smem_u32(&bar_full[i]), (u - (u / k_blocks) * k_blocks) * BK, 0);
		}
	}
	if (warp == 1)
	{
		tmem_alloc(smem_u32(&tmem_slot), TMEM_COLS);
		tmem_relinquish();
	}
	tc_fence_before();
	__syncthreads();
	tc_fence_after();
	const uint32_t tmem_base = tmem_slot;

	if (warp == 0)
	{
		if (lane == 0)
		{
			int stage = n_first == STAGES ? 0 : n_first;
			uint32_t phase = n_first == STAGES ? 1u : 0u;
			for (int u = u_begin + n_first; u < u_end; ++u)
			{
				if (!mbar_wait(smem_u32(&bar_empty[stage]), phase ^ 1u, abortp))
				{
					report_timeout(err_word, kErrProducerWait);
					goto role_done;
				}
				load_unit(u, stage, false);
				if (++stage == STAGES) { stage = 0; phase ^= 1u; }
			}
		}
	}
	else if (warp == 1)
	{
		if (lane == 0)
		{
			constexpr uint32_t idesc = make_idesc_f16(BM, BN, B_MN);
			int stage = 0;
			uint32_t phase = 0;
			int acc = 0;
			uint32_t acc_phase = 0;
			for (int u = u_begin; u < u_end;)
			{
				const int tile = u / k_blocks;
				const int seg_end = min(u_end, (tile + 1) * k_blocks);
				if (!mbar_wait(smem_u32(&bar_tempty[acc]), acc_phase ^ 1u, abortp))
				{
					report_timeout(err_word, kErrMmaWaitTmem);
					goto role_done;
				}
				tc_fence_after();
				const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
				for (int v = u; v < seg_end; ++v)
				{
					if (!mbar_wait(smem_u32(&bar_full[stage]), phase, abortp))
					{
						report_timeout(err_word, kErrMmaWaitFull);
						goto role_done;
					}
					tc_fence_after();
					const uint32_t a_s = ring + stage * STAGE_BYTES;
					const uint32_t b_s = a_s + A_BYTES;
					const uint64_t a_desc = make_smem_desc_sw128(a_s, 16, 1024);
					const uint64_t b_desc = B_MN ? make_smem_desc_sw128(b_s, BK * 128, 1024) : make_smem_desc_sw128(b_s, 16, 1024);
#pragma unroll
					for (int k = 0; k < BK / 16; ++k)
					{
						const uint64_t a_k = a_desc + static_cast<uint64_t>(k * 2);
						const uint64_t b_k = b_desc + static_cast<uint64_t>(B_MN ? k * 128 : k * 2);
						mma_f16_ss(d_tmem, a_k, b_k, idesc, (v != u || k != 0) ? 1u : 0u);
					}
					mma_commit(smem_u32(&bar_empty[stage]));
					if (++stage == STAGES) { stage = 0; phase ^= 1u; }
				}
				mma_commit(smem_u32(&bar_tfull[acc]));
				if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
				u = seg_end;
			}
		}
	}
	else
	{
		const int q = warp & 3;  // TMEM lane quadrant this warp may read
		const bool owns_rows = q * 32 < M;  // warp-uniform: quadrants past M hold nothing to keep
		const uint32_t stg_s = ring + STAGES * STAGE_BYTES + (q < R::STG_WARPS ? q : 0) * (2 * STG_BYTES);
		uint8_t* stg = smem_raw + (stg_s - smem_u32(smem_raw));
		if (lane == 0) prefetch_tmap(&tmP);
		pdl_wait();  // the partial buffer may still be read by the kernel before this one
		int acc = 0;
		uint32_t acc_phase = 0;
		uint32_t nchunk = 0;
		for (int u = u_begin; u < u_end;)
		{
			const int tile = u / k_blocks;
			const int seg_end = min(u_end, (tile + 1) * k_blocks);
			const int slice = static_cast<int>(blockIdx.x) - cta_of_unit(static_cast<int64_t>(tile) * k_blocks, gridDim.x, total_units);
			if (!mbar_wait(smem_u32(&bar_tfull[acc]), acc_phase, abortp))
			{
				if (lane == 0) report_timeout(err_word, kErrEpilogueWait);
				goto role_done;
			}
			tc_fence_after();
			if (owns_rows)
			{
				const uint32_t t_base = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(acc * BN);
#pragma unroll 1
				for (int c = 0; c < BN / 64; ++c)
				{
					uint32_t r[2][32];
					tmem_ld_32x32(t_base + static_cast<uint32_t>(c * 64), r[0]);
					tmem_ld_32x32(t_base + static_cast<uint32_t>(c * 64 + 32), r[1]);
					tmem_ld_wait();
#pragma unroll
					for (int hh = 0; hh < 2; ++hh)
					{
						// the staging buffer about to be rewritten must have been read by its store
						if (lane == 0) bulk_wait_group_read<1>();
						__syncwarp();
						const uint32_t buf = nchunk & 1u;
						uint8_t* srow = stg + buf * STG_BYTES + lane * 128;
#pragma unroll
						for (int v = 0; v < 8; ++v)
							*reinterpret_cast<uint4*>(srow + ((v ^ (lane & 7)) << 4)) =
								make_uint4(r[hh][v * 4], r[hh][v * 4 + 1], r[hh][v * 4 + 2], r[hh][v * 4 + 3]);
						fence_proxy_async_smem();
						__syncwarp();
						if (lane == 0)
						{
							// rows past M of this slice are clipped by the 3-D map [slices, M, 256]
							tma_store_3d(&tmP, stg_s + buf * STG_BYTES, c * 64 + hh * 32, q * 32, tile * max_seg + slice);
							bulk_commit_group();
						}
						++nchunk;
					}
				}
			}
			tc_fence_before();
			__syncwarp();
			if (lane == 0) mbar_arrive(smem_u32(&bar_tempty[acc]));
			if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
			u = seg_end;
		}
		if (lane == 0) bulk_wait_group<0>();  // stores must have left shared memory before the CTA exits
	}

role_done:
	__syncwarp();
	if (*abortp)
	{
		// give copies and MMAs already in flight time to land before shared and tensor memory are released
		for (int i = 0; i < 2000; ++i) __nanosleep(1000);
	}
	tc_fence_before();
	__syncthreads();
	if (warp == 1)
	{
		tc_fence_after();
		tmem_dealloc(tmem_base, TMEM_COLS);
	}
}

// ---- consumers of the partial tiles ----------------------------------------------------------------------------------
// One thread per (row, 4 columns): the slices of its float4 are fetched in batches of 8 independent loads and added in slice
// order (a fixed order: the result does not depend on scheduling).
__device__ __forceinline__ float4 sum_slices4(const float* __restrict__ part, int r, int col, int M, int k_blocks, int total_units, int grid,
	int max_seg)
{
	using namespace dgemm;
	const int tile = col / BN;
	const int first = cta_of_unit(static_cast<int64_t>(tile) * k_blocks, grid, total_units);
	const int nseg = cta_of_unit(static_cast<int64_t>(tile + 1) * k_blocks - 1, grid, total_units) - first + 1;
	const float* p = part + ((static_cast<int64_t>(tile) * max_seg) * M + r) * BN + (col - tile * BN);
	const int64_t seg_stride = static_cast<int64_t>(M) * BN;
	float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
	for (int s0 = 0; s0 < nseg; s0 += 8)
	{
		float4 t[8];
#pragma unroll
		for (int i = 0; i < 8; ++i)
			t[i] = s0 + i < nseg ? *reinterpret_cast<const float4*>(p + (s0 + i) * seg_stride) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
		for (int i = 0; i < 8; ++i)
		{
			a.x += t[i].x; a.y += t[i].y; a.z += t[i].z; a.w += t[i].w;
		}
	}
	return a;
}

struct alignas(8) Half4
{
	__half2 h[2];
};
__device__ __forceinline__ Half4 pack4(float a, float b, float c, float d)
{
	Half4 v;
	v.h[0] = __floats2half2_rn(a, b);
	v.h[1] = __floats2half2_rn(c, d);
	return v;
}
__device__ __forceinline__ void unpack4(const Half4& v, float* f)
{
	const float2 a = __half22float2(v.h[0]), b = __half22float2(v.h[1]);
	f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}

// in_proj consumer. Row r = blockIdx.y, 4 columns per thread. Columns [conv_lo, conv_lo + conv_dim) additionally go through
// the rolling causal conv1d update (state [M, conv_dim, W-1] shifted by one, y = silu(bias + sum_k w[k] * window[k]), the
// arithmetic of conv1d_update_kernel on the f16-rounded projection) and are written to xbc[M, conv_dim]; every column is
// written to zx[M, ldz] as f16.
__global__ void __launch_bounds__(256, 5) streamk_reduce_conv_kernel(const float* __restrict__ part, __half* __restrict__ zx, int64_t ldz,
	int M, int N, int k_blocks, int total_units, int grid, int max_seg, int conv_lo, int conv_dim, int W,
	__half* __restrict__ conv_state, const __half* __restrict__ conv_w, const __half* __restrict__ conv_b, __half* __restrict__ xbc)
{
	pdl_launch_dependents();
	const int r = blockIdx.y;
	const int col = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
	const bool live = col < N;
	const bool conv = live && col >= conv_lo && col < conv_lo + conv_dim;
	const int ch = col - conv_lo;
	const int SW = W - 1;
	// weights do not depend on the kernel before this one
	float w[16], bias[4];
	if (conv && W == 4)
	{
		const Half8 w0 = *reinterpret_cast<const Half8*>(conv_w + static_cast<int64_t>(ch) * 4);
		const Half8 w1 = *reinterpret_cast<const Half8*>(conv_w + static_cast<int64_t>(ch) * 4 + 8);
		unpack8(w0, w);
		unpack8(w1, w + 8);
		unpack4(*reinterpret_cast<const Half4*>(conv_b + ch), bias);
	}
	pdl_wait();
	if (!live) return;
	__half* st = conv_state + (static_cast<int64_t>(r) * conv_dim + ch) * SW;
	Half4 sv[3];
	if (conv && W == 4)
	{
#pragma unroll
		for (int i = 0; i < 3; ++i) sv[i] = *reinterpret_cast<const Half4*>(st + i * 4);  // 4 channels x 3 state values: 24 bytes
	}
	const float4 acc4 = sum_slices4(part, r, col, M, k_blocks, total_units, grid, max_seg);
	const Half4 h = pack4(acc4.x, acc4.y, acc4.z, acc4.w);
	*reinterpret_cast<Half4*>(zx + static_cast<int64_t>(r) * ldz + col) = h;
	if (!conv) return;
	float x[4];
	unpack4(h, x);  // the conv sees the projection as the f16 tensor it is between the two operators
	float y[4];
	if (W == 4)
	{
		float s[12], ns[12];
#pragma unroll
		for (int i = 0; i < 3; ++i) unpack4(sv[i], s + i * 4);
#pragma unroll
		for (int j = 0; j < 4; ++j)
		{
			float acc = 0.f;
#pragma unroll
			for (int k = 0; k < 3; ++k) acc += w[j * 4 + k] * s[j * 3 + k];
			acc += w[j * 4 + 3] * x[j];
			acc += bias[j];
			y[j] = silu_f32(acc);
			ns[j * 3] = s[j * 3 + 1];
			ns[j * 3 + 1] = s[j * 3 + 2];
			ns[j * 3 + 2] = x[j];
		}
#pragma unroll
		for (int i = 0; i < 3; ++i) *reinterpret_cast<Half4*>(st + i * 4) = pack4(ns[i * 4], ns[i * 4 + 1], ns[i * 4 + 2], ns[i * 4 + 3]);
	}
	else
	{
		for (int j = 0; j < 4; ++j)
		{
			__half* sj = st + j * SW;
			const __half* wj = conv_w + static_cast<int64_t>(ch + j) * W;
			float acc = 0.f;
			for (int k = 0; k < SW; ++k) acc += ldf(wj + k) * ldf(sj + k);
			acc += ldf(wj + SW) * x[j];
			acc += ldf(conv_b + ch + j);
			y[j] = silu_f32(acc);
			for (int k = 0; k + 1 < SW; ++k) sj[k] = sj[k + 1];
			if (SW > 0) stf(sj + SW - 1, x[j]);
		}
	}
	*reinterpret_cast<Half4*>(xbc + static_cast<int64_t>(r) * conv_dim + ch) = pack4(y[0], y[1], y[2], y[3]);
}

// out_proj consumer: many slices per tile (K is long, N short), so the slice loads are spread over the CTA as well. One CTA
// per (256-column tile, row): 64 column quads x 4 slice groups; group g adds slices g, g+4, ... of its quad, the four group
// sums are combined in group order through shared memory (again a fixed order), and warp 0 finishes 8 columns per lane.
// With sumsq != nullptr the row is multiplied by rsqrt(sum_j sumsq[r, j] / norm_dim + eps): the RMSNorm scale factored out
// of the projection (the projection's input then carries y * silu(z) * weight un-normalised).
__global__ void __launch_bounds__(256) streamk_reduce_scale_kernel(const float* __restrict__ part, __half* __restrict__ out, int64_t ldo,
	int M, int N, int k_blocks, int total_units, int grid, int max_seg, const float* __restrict__ sumsq, int nsumsq, float inv_norm_dim,
	float eps, const __half* __restrict__ residual, int64_t ldr)
{
	using namespace dgemm;
	__shared__ float4 sm[4][64];
	pdl_launch_dependents();
	pdl_wait();
	const int tile = blockIdx.x, r = blockIdx.y;
	const int quad = threadIdx.x & 63, sg = threadIdx.x >> 6;
	const int first = cta_of_unit(static_cast<int64_t>(tile) * k_blocks, grid, total_units);
	const int nseg = cta_of_unit(static_cast<int64_t>(tile + 1) * k_blocks - 1, grid, total_units) - first + 1;
	const float* p = part + ((static_cast<int64_t>(tile) * max_seg) * M + r) * BN + quad * 4;
	const int64_t seg_stride = static_cast<int64_t>(M) * BN;
	float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
	for (int s = sg; s < nseg; s += 4)
	{
		const float4 t = *reinterpret_cast<const float4*>(p + s * seg_stride);
		a.x += t.x; a.y += t.y; a.z += t.z; a.w += t.w;
	}
	sm[sg][quad] = a;
	const int lane = threadIdx.x;
	float sc = 1.f;
	if (lane < 32 && sumsq)
	{
		float v = 0.f;
		for (int j = lane; j < nsumsq; j += 32) v += sumsq[static_cast<int64_t>(r) * nsumsq + j];
		sc = rsqrtf(warp_sum(v) * inv_norm_dim + eps);
	}
	__syncthreads();
	const int col = tile * BN + lane * 8;
	if (lane >= 32 || col >= N) return;
	float f[8];
#pragma unroll
	for (int hh = 0; hh < 2; ++hh)
	{
		float4 t = sm[0][2 * lane + hh];
#pragma unroll
		for (int g = 1; g < 4; ++g)
		{
			const float4 v = sm[g][2 * lane + hh];
			t.x += v.x; t.y += v.y; t.z += v.z; t.w += v.w;
		}
		f[4 * hh] = t.x * sc; f[4 * hh + 1] = t.y * sc; f[4 * hh + 2] = t.z * sc; f[4 * hh + 3] = t.w * sc;
	}
	if (residual != nullptr)  // the residual stream of the layer around the mixer, added before the one rounding
	{
		float rv[8];
		unpack8(*reinterpret_cast<const Half8*>(residual + static_cast<int64_t>(r) * ldr + col), rv);
#pragma unroll
		for (int j = 0; j < 8; ++j) f[j] += rv[j];
	}
	*reinterpret_cast<Half8*>(out + static_cast<int64_t>(r) * ldo + col) = pack8(f);
}

// ---- host side -------------------------------------------------------------------------------------------------------

struct StreamKPlan
{
	int k_blocks, n_tiles, total, grid, max_seg;
};

static StreamKPlan streamk_plan(int64_t K, int64_t N)
{
	StreamKPlan p;
	p.k_blocks = static_cast<int>(cdiv(K, dgemm::BK));
	p.n_tiles = static_cast<int>(cdiv(N, dgemm::BN));
	p.total = p.k_blocks * p.n_tiles;
	p.grid = p.total < kNumSMs ? p.total : kNumSMs;
	p.max_seg = 1;
	for (int t = 0; t < p.n_tiles; ++t)
	{
		const int first = dgemm::cta_of_unit(static_cast<int64_t>(t) * p.k_blocks, p.grid, p.total);
		const int last = dgemm::cta_of_unit(static_cast<int64_t>(t + 1) * p.k_blocks - 1, p.grid, p.total);
		if (last - first + 1 > p.max_seg) p.max_seg = last - first + 1;
	}
	return p;
}

bool decode_linear_applies(int dtype, int64_t M, int64_t K, int64_t N)
{
	return dtype == B200_F16 && M >= 1 && M <= 128 && K % 8 == 0 && N % 8 == 0 && cdiv(N, dgemm::BN) * 2 <= kNumSMs && K >= 4 * dgemm::BK &&
		cdiv(K, dgemm::BK) * cdiv(N, dgemm::BN) < (1 << 20);
}

size_t decode_linear_partial_bytes(int64_t M, int64_t K, int64_t N)
{
	const StreamKPlan p = streamk_plan(K, N);
	return align_up(static_cast<size_t>(p.n_tiles) * p.max_seg * M * dgemm::BN * sizeof(float), 256);
}

template <int B_MN, int A_ROWS>
static int launch_streamk(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmP, int M, const StreamKPlan& p, cudaStream_t st)
{
	using R = dgemm::Ring<A_ROWS>;
	static bool smem_ok[64] = {};
	B200_CUDA_TRY(allow_dynamic_smem(gemm_f16_streamk_kernel<B_MN, A_ROWS>, R::SMEM_BYTES, smem_ok));
	B200_CUDA_TRY(launch_chained(pdl_enabled(), gemm_f16_streamk_kernel<B_MN, A_ROWS>, dim3(p.grid), dim3(dgemm::THREADS), R::SMEM_BYTES, st,
		tmA, tmB, tmP, M, p.k_blocks, p.total, p.max_seg, device_error_word()));
	return B200_OK;
}

// The stream-K GEMM alone: fills `part` for the problem X[M,K] (row stride ldx) . W.
static int decode_gemm(const void* x, int64_t ldx, const void* w, int w_layout, int64_t M, int64_t K, int64_t N, float* part,
	StreamKPlan* plan, cudaStream_t st)
{
	using namespace dgemm;
	if (ldx % 8 != 0 || !aligned16(x) || !aligned16(w) || !aligned16(part)) return B200_ERR_MISALIGNED;
	const bool half_rows = M <= 64;
	CUtensorMap tmA, tmB;
	int rc = tmap_2d_f16(&tmA, x, static_cast<uint64_t>(M), static_cast<uint64_t>(K), static_cast<uint64_t>(ldx), BK, half_rows ? 64 : BM);
	if (rc) return rc;
	if (w_layout == B200_W_NK)
		rc = tmap_2d_f16(&tmB, w, static_cast<uint64_t>(N), static_cast<uint64_t>(K), static_cast<uint64_t>(K), BK, BN);
	else if (w_layout == B200_W_KN)
		rc = tmap_2d_f16(&tmB, w, static_cast<uint64_t>(K), static_cast<uint64_t>(N), static_cast<uint64_t>(N), 64, BK);
	else
		return B200_ERR_UNSUPPORTED;
	if (rc) return rc;
	*plan = streamk_plan(K, N);
	// partial tiles as a 3-D fp32 tensor [tile * max_seg + slice][M][256]: stores of 32-row boxes are clipped at M
	CUtensorMap tmP;
	rc = tmap_3d_f32(&tmP, part, BN, static_cast<uint64_t>(M), static_cast<uint64_t>(plan->n_tiles) * plan->max_seg, BN,
		static_cast<uint64_t>(M) * BN, 32, 32);
	if (rc) return rc;
	const int m = static_cast<int>(M);
	if (w_layout == B200_W_NK)
		return half_rows ? launch_streamk<0, 64>(tmA, tmB, tmP, m, *plan, st) : launch_streamk<0, 128>(tmA, tmB, tmP, m, *plan, st);
	return half_rows ? launch_streamk<1, 64>(tmA, tmB, tmP, m, *plan, st) : launch_streamk<1, 128>(tmA, tmB, tmP, m, *plan, st);
}

// in_proj of a decode step followed by the rolling conv update of its xBC columns (see streamk_reduce_conv_kernel).
int decode_in_proj_conv(const void* x, int64_t ldx, const void* w, int w_layout, void* zx, int64_t ldz, int64_t M, int64_t K, int64_t N,
	int64_t conv_lo, int64_t conv_dim, int conv_width, void* conv_state, const void* conv_w, const void* conv_b, void* xbc, float* part,
	cudaStream_t st)
{
	if (conv_lo % 4 != 0 || conv_dim % 4 != 0 || N % 4 != 0 || ldz % 4 != 0 || !aligned16(zx) || !aligned16(conv_state) || !aligned16(conv_w) ||
		!aligned16(conv_b) || !aligned16(xbc))
		return B200_ERR_MISALIGNED;
	if (conv_width < 1 || conv_lo + conv_dim > N) return B200_ERR_BAD_SHAPE;
	StreamKPlan p;
	const int rc = decode_gemm(x, ldx, w, w_layout, M, K, N, part, &p, st);
	if (rc) return rc;
	const dim3 g(static_cast<unsigned>(cdiv(N / 4, 256)), static_cast<unsigned>(M));
	B200_CUDA_TRY(launch_chained(pdl_enabled(), streamk_reduce_conv_kernel, g, dim3(256), 0, st, static_cast<const float*>(part),
		static_cast<__half*>(zx), ldz, static_cast<int>(M), static_cast<int>(N), p.k_blocks, p.total, p.grid, p.max_seg,
		static_cast<int>(conv_lo), static_cast<int>(conv_dim), conv_width, static_cast<__half*>(conv_state),
		static_cast<const __half*>(conv_w), static_cast<const __half*>(conv_b), static_cast<__half*>(xbc)));
	return B200_OK;
}

// out_proj of a decode step; sumsq [M, nsumsq] (or nullptr) carries the partial sums of squares of the RMSNorm; residual
// [M, >= N] (or nullptr) is added to the result.
int decode_out_proj_scale(const void* x, int64_t ldx, const void* w, int w_layout, void* out, int64_t ldo, int64_t M, int64_t K, int64_t N,
	const float* sumsq, int nsumsq, int64_t norm_dim, float eps, float* part, cudaStream_t st, const void* residual, int64_t ldr)
{
	if (ldo % 8 != 0 || !aligned16(out)) return B200_ERR_MISALIGNED;
	if (residual && (ldr % 8 != 0 || !aligned16(residual))) return B200_ERR_MISALIGNED;
	StreamKPlan p;
	const int rc = decode_gemm(x, ldx, w, w_layout, M, K, N, part, &p, st);
	if (rc) return rc;
	const dim3 g(static_cast<unsigned>(p.n_tiles), static_cast<unsigned>(M));
	// normal launch: measured slower when this kernel's CTAs are resident (waiting) while the projection before it runs
	B200_CUDA_TRY(launch_chained(false, streamk_reduce_scale_kernel, g, dim3(256), 0, st, static_cast<const float*>(part),
		static_cast<__half*>(out), ldo, static_cast<int>(M), static_cast<int>(N), p.k_blocks, p.total, p.grid, p.max_seg, sumsq, nsumsq,
		1.0f / static_cast<float>(norm_dim), eps, static_cast<const __half*>(residual), ldr));
	return B200_OK;
}

}  // namespace b200
