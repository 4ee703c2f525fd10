// SSD chunked scan as ONE tensor-core kernel for f16 activations: chunk states, state passing and chunk scan in a single
// pass over the sequence (the dt stage, softplus and in-chunk cumulative sums, still runs before it).
//
// One CTA owns one (batch, head) pair and walks its sequence in blocks of 128 tokens, carrying the [P x N] state in registers
// (fp32). Per block, with l, s = token inside the block, dA = the cumulative sum of dt*A up to and including a token:
//   CB  = C . B^T                                              tcgen05, M = l (128), N = s (128), K = n
//   S   = CB o exp(dA[l] - dA[s]) dt[s] o (s <= l), S[l,l] += D  CUDA cores: TMEM -> f16 tile in shared memory
//   Y   = S . X  +  rowdec[l] * (C . prev^T)                   tcgen05, M = l, N = p, K = s and K = n; rowdec = exp(dA[l] - dA[before block])
//   ST  = X^T . (w o B),  w[l] = exp(dA[last] - dA[l]) dt[l]    tcgen05, M = p, N = n, K = l (B is scaled in place once CB is done)
//   state <- exp(dA[last] - dA[before block]) state + ST        registers; its f16 copy is the `prev` operand of the next block
// which is the arithmetic of mamba_chunk_scan_combined_ref (scripts/zamba2/mamba_chunk_scan_comb.py:51-160) with the chunk
// states never leaving the SM: x, B and C are read once, y is written once, and nothing else touches HBM. The result does not
// depend on how the sequence is cut into blocks, so the public `chunk` (128 or 256) only fixes where the dt stage restarts its
// cumulative sums.
// Roles: eight compute warps (TMEM lane quadrant x column half) and one producer warp whose lane 0 issues every TMA copy and
// every MMA; they meet only at mbarriers. A block's chain is: tiles land -> CB -> S -> MMAs -> tiles of the next block (the
// buffers are single: 104 KiB of shared memory and 256 tensor-memory columns per CTA, so that two CTAs share an SM); the
// y epilogue and the state update of a block run while the next block's tiles are on their way, and the next tiles are
// requested into L2 one block ahead.
// Every decay is the exponential of a non-positive difference. Every mbarrier wait is bounded; on a timeout the CTA records a
// code, drains and frees its tensor memory.
#include <cstdlib>
#include <type_traits>

#include "ssd_common.cuh"
#include "tcgen05.cuh"

namespace b200 {

using namespace tc;

namespace sfused {
constexpr int NCW = 8;                   // compute warps: 4 TMEM lane quadrants x 2 column halves
constexpr int THREADS = (NCW + 1) * 32;  // + the producer warp
constexpr int QI = 128;                  // tokens per block
constexpr int TILE = QI * 128;           // a [128 rows][64 f16] tile: 16 KiB
constexpr int OFF_C = 0;                 // C  [128 l][64 n]   K-major A operand of CB and of C.prev^T
constexpr int OFF_B = OFF_C + TILE;      // B  [128 s][64 n]   K-major B operand of CB; scaled rows: MN-major B operand of ST
constexpr int OFF_X = OFF_B + TILE;      // X  [128 s][64 p]   MN-major B operand of S.X and MN-major A operand of ST
constexpr int OFF_S = OFF_X + TILE;      // S  2 x [128 l][64 s]  K-major A operand (one tile per 64-wide K-block)
constexpr int OFF_P = OFF_S + 2 * TILE;  // prev [64 p][64 n]  K-major B operand of C.prev^T
constexpr int OFF_Y = OFF_P + TILE / 2;  // y staging [128 l][64 p], 128-byte swizzled like the TMA store expects
constexpr int TOTAL = OFF_Y + TILE + 1024;
constexpr uint32_t TMEM_COLS = 256;      // CB [0,128) (ST reuses [0,64) once S is written) | Y [128,192) | C.prev^T [192,256)
constexpr float kLog2e = 1.4426950408889634f;
static_assert(2 * (TOTAL + 4096) <= 232448, "two CTAs must fit one SM");
}  // namespace sfused

__device__ __forceinline__ float ex2f(float v)
{
	float r;
	asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v));
	return r;
}

__device__ __forceinline__ void named_barrier_sync(int id, int nthreads)
{
	asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// VARLEN: the batch is a packed run of sequences (rows cu[s] .. cu[s+1]-1 of one [tokens, features] tensor); CTA = (sequence, head).
// The dt stage then writes its rows per 128-token block of every sequence (block coff[s] + j of head h at ((h * nblk) + coff[s] + j) * 128,
// cumulative sums restarting at every block, dt = 0 past the end of a sequence). Rows that a tile holds past the end of its
// sequence belong to the next one; they carry dt = 0 in this sequence's scalars, which zeroes their columns of S and their
// rows of the state update, and their rows of y are not stored.
template <bool VARLEN>
__global__ void __launch_bounds__(sfused::THREADS, 2) ssd_fused_tc_kernel(const __grid_constant__ CUtensorMap tmX,
	const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmY,
	const float* __restrict__ D, const float* __restrict__ dt, const float* __restrict__ dacs,
	const float* init, float* fin /* may alias init: every thread reads its slice first */, int64_t seqlen, int H, int G, int Q, int nchunks,
	uint32_t* err_word, const int* __restrict__ cu /* VARLEN: token offsets [nseq + 1] */, const int* __restrict__ coff /* VARLEN: block offsets */,
	int nblk /* VARLEN: 128-token blocks of all sequences */, __half* __restrict__ yv /* VARLEN: y, for the ragged last block */, int64_t ys)
{
	using namespace sfused;
	extern __shared__ uint8_t smem_raw[];
	// producer -> compute: bar_cb (CB in tensor memory), bar_y (S.X and C.prev^T done), bar_st (state MMAs done; also frees the tiles)
	// compute -> producer: bar_s (S tile and scaled B written: one arrival per compute warp), bar_epi (block's results read out of
	// tensor memory, y staged, prev written: one arrival per compute warp); bar_in: the TMA loads of a block
	__shared__ uint64_t bar_in, bar_cb, bar_y, bar_st, bar_s, bar_epi;
	__shared__ uint32_t tmem_slot;
	__shared__ int abort_flag;
	__shared__ __align__(16) float sc_dA2[2][QI], sc_q2[2][QI], sc_cf[2][QI], sc_rowdec[2][QI], sc_w[2][QI];  // sc_cf: see below
	__shared__ float sc_dec[2];

	const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
	uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
	const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
	const int q = warp & 3;        // TMEM lane quadrant this warp may read
	const int half = (warp >> 2) & 1;  // which 64-wide K-block of S / which 32 columns of an accumulator this warp owns
	const int r = q * 32 + lane;   // row (l, or p for the state) inside the block
	const int h = static_cast<int>(blockIdx.x % H);
	const int64_t bs_ = blockIdx.x / H;               // batch entry, or sequence of a packed batch
	const int64_t b = VARLEN ? 0 : bs_;               // third TMA coordinate
	const int tok0 = VARLEN ? cu[bs_] : 0;            // first row of the sequence inside the packed tensor
	const int len = VARLEN ? cu[bs_ + 1] - tok0 : 0;  // VARLEN: tokens of this sequence
	const int g = h / (H / G);
	const int nsub = VARLEN ? (len + QI - 1) / QI : nchunks * (Q / QI);
	const int64_t bh = bs_ * H + h;
	const int64_t srow0 = VARLEN ? (static_cast<int64_t>(h) * nblk + coff[bs_]) * QI : bh * nchunks * static_cast<int64_t>(Q);
	const float* dacs_bh = dacs + srow0;
	const float* dt_bh = dt + srow0;
	volatile int* abortp = &abort_flag;
	const uint32_t in = smem_u32(&bar_in), cbb = smem_u32(&bar_cb), yb = smem_u32(&bar_y), stb = smem_u32(&bar_st),
		sb = smem_u32(&bar_s), epib = smem_u32(&bar_epi);

	if (threadIdx.x == 0)
	{
		abort_flag = 0;
		mbar_init(in, 1);
		mbar_init(cbb, 1);
		mbar_init(yb, 1);
		mbar_init(stb, 1);
		mbar_init(sb, NCW);
		mbar_init(epib, NCW);
		fence_mbar_init();
		prefetch_tmap(&tmX); prefetch_tmap(&tmB); prefetch_tmap(&tmC); prefetch_tmap(&tmY);
	}
	if (warp == 0)
	{
		tmem_alloc(smem_u32(&tmem_slot), TMEM_COLS);
		tmem_relinquish();
	}
	if (warp < NCW)
	{
		// the parts of S above the diagonal stay zero for the whole kernel
		Half8 zero;
#pragma unroll
		for (int e = 0; e < 4; ++e) zero.h[e] = __floats2half2_rn(0.f, 0.f);
		for (int i = threadIdx.x; i < 2 * TILE / 16; i += NCW * 32) *reinterpret_cast<Half8*>(gen + OFF_S + i * 16) = zero;
	}
	tc_fence_before();
	__syncthreads();
	tc_fence_after();
	const uint32_t tmem_base = tmem_slot;

	if (warp == NCW)
	{
		// ================================= producer warp: every TMA copy and every MMA =================================
		if (lane == 0)
		{
			uint32_t fail = 0;
			// the three tiles of block j (one 128-row box each; rows past the end of the sequence arrive as zeros), and a request
			// that brings the tiles of block j+1 into L2 meanwhile: a block's loads start only when the MMAs of the block before
			// have released the buffers, so their latency is on the critical path of every block
			auto issue_loads = [&](int j) {
				const int t0 = tok0 + j * QI;
				mbar_arrive_expect_tx(in, 3 * TILE);
				tma_load_3d(base + OFF_C, &tmC, in, g * 64, t0, static_cast<int>(b));
				tma_load_3d(base + OFF_B, &tmB, in, g * 64, t0, static_cast<int>(b));
				tma_load_3d(base + OFF_X, &tmX, in, h * 64, t0, static_cast<int>(b));
				if (j + 1 < nsub)
				{
					tma_prefetch_3d(&tmC, g * 64, t0 + QI, static_cast<int>(b));
					tma_prefetch_3d(&tmB, g * 64, t0 + QI, static_cast<int>(b));
					tma_prefetch_3d(&tmX, h * 64, t0 + QI, static_cast<int>(b));
				}
			};
			auto store_y = [&](int j) {
				const int t0 = tok0 + j * QI;
				if (VARLEN)
				{
					// a whole block goes out as two boxes; the ragged last block was written row by row by the compute warps
					if ((j + 1) * QI <= len)
					{
						tma_store_3d(&tmY, base + OFF_Y, h * 64, t0, 0);
						tma_store_3d(&tmY, base + OFF_Y + 8192, h * 64, t0 + 64, 0);
					}
					bulk_commit_group();
					return;
				}
				// rows past the end of the sequence are clipped by the store; a box that starts past it is not issued at all
				if (t0 < seqlen) tma_store_3d(&tmY, base + OFF_Y, h * 64, t0, static_cast<int>(b));
				if (t0 + 64 < seqlen) tma_store_3d(&tmY, base + OFF_Y + 8192, h * 64, t0 + 64, static_cast<int>(b));
				bulk_commit_group();
			};
			constexpr uint32_t idesc_cb = make_idesc_f16(QI, QI, 0);
			constexpr uint32_t idesc_y = make_idesc_f16(QI, 64, 1);      // B operand (x) MN-major
			constexpr uint32_t idesc_z = make_idesc_f16(QI, 64, 0);
			constexpr uint32_t idesc_st = make_idesc_f16(128, 64, 1, 1);  // A (x) and B (scaled B) MN-major
			const uint64_t c_desc = make_smem_desc_sw128(base + OFF_C, 16, 1024);
			const uint64_t bk_desc = make_smem_desc_sw128(base + OFF_B, 16, 1024);
			const uint64_t p_desc = make_smem_desc_sw128(base + OFF_P, 16, 1024);
			if (nsub > 0) issue_loads(0);
			for (int j = 0; j < nsub && fail == 0; ++j)
			{
				const uint32_t par = static_cast<uint32_t>(j) & 1u;
				if (!mbar_wait(in, par, abortp)) { fail = kErrProducerWait; break; }
				if (j > 0)
				{
					// block j-1 has been read out of tensor memory (its CB / ST columns and accumulators may be overwritten), its prev
					// tile is written and its y tile is staged
					if (!mbar_wait(epib, par ^ 1u, abortp)) { fail = kErrProducerWait; break; }
				}
				tc_fence_after();
#pragma unroll
				for (int k = 0; k < 4; ++k)
					mma_f16_ss(tmem_base, c_desc + static_cast<uint64_t>(k * 2), bk_desc + static_cast<uint64_t>(k * 2), idesc_cb, k != 0 ? 1u : 0u);
				mma_commit(cbb);
				if (j > 0) store_y(j - 1);  // after the CB issue: the compute warps wait for CB, nobody waits for the store
				if (!mbar_wait(sb, par, abortp)) { fail = kErrMmaWaitFull; break; }
				tc_fence_after();
				bulk_wait_group_read<0>();  // the previous y store has read the staging tile that this block's epilogue rewrites
#pragma unroll
				for (int kb = 0; kb < 2; ++kb)
				{
					const uint64_t a_desc = make_smem_desc_sw128(base + OFF_S + kb * TILE, 16, 1024);
					const uint64_t b_desc = make_smem_desc_sw128(base + OFF_X + kb * 8192, 8192, 1024);
#pragma unroll
					for (int k = 0; k < 4; ++k)
						mma_f16_ss(tmem_base + 128u, a_desc + static_cast<uint64_t>(k * 2), b_desc + static_cast<uint64_t>(k * 128), idesc_y,
							(kb | k) != 0 ? 1u : 0u);
				}
#pragma unroll
				for (int k = 0; k < 4; ++k)
					mma_f16_ss(tmem_base + 192u, c_desc + static_cast<uint64_t>(k * 2), p_desc + static_cast<uint64_t>(k * 2), idesc_z, k != 0 ? 1u : 0u);
				mma_commit(yb);
#pragma unroll
				for (int kb = 0; kb < 2; ++kb)
				{
					// M = 128 although the state has 64 rows (p): rows 64-127 multiply whatever follows the x tile and are never read
					const uint64_t a_desc = make_smem_desc_sw128(base + OFF_X + kb * 8192, 8192, 1024);
					const uint64_t b_desc = make_smem_desc_sw128(base + OFF_B + kb * 8192, 8192, 1024);
#pragma unroll
					for (int k = 0; k < 4; ++k)
						mma_f16_ss(tmem_base, a_desc + static_cast<uint64_t>(k * 128), b_desc + static_cast<uint64_t>(k * 128), idesc_st,
							(kb | k) != 0 ? 1u : 0u);
				}
				mma_commit(stb);
				if (j + 1 < nsub)
				{
					// the next block's tiles go where this block's are: every MMA that reads them must have completed
					if (!mbar_wait(stb, par, abortp)) { fail = kErrMmaWaitTmem; break; }
					issue_loads(j + 1);
				}
			}
			if (fail == 0 && nsub > 0)
			{
				if (mbar_wait(epib, static_cast<uint32_t>(nsub - 1) & 1u, abortp)) store_y(nsub - 1);
				else fail = kErrProducerWait;
			}
			if (fail != 0) report_timeout(err_word, fail);
			bulk_wait_group<0>();  // stores must have left shared memory before the CTA exits
		}
	}
	else
	{
		// ================================= compute warps =================================================================
		const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
		const float dh = D ? __ldg(D + h) : 0.f;
		bool dead = false;  // a wait gave up: keep walking the loop (the barriers still need this warp) but do no work

		// per-row scalars of the next block, fetched one block ahead (warps 0-3: thread = row)
		float nx_dA = 0.f, nx_dt = 0.f, nx_last = 0.f, nx_base = 0.f;
		auto fetch_scalars = [&](int j) {
			if (warp < 4 && j < nsub)
			{
				const int o = j * QI;
				nx_dA = __ldg(dacs_bh + o + r);
				nx_dt = __ldg(dt_bh + o + r);
				nx_last = __ldg(dacs_bh + o + QI - 1);
				// the cumulative sums restart at every public chunk (at every block of a packed batch)
				nx_base = !VARLEN && (o % Q) != 0 ? __ldg(dacs_bh + o - 1) : 0.f;
			}
		};
		fetch_scalars(0);

		// the state: thread (q < 2) owns row p = r, columns n = half*32 .. +31
		float state[32];
#pragma unroll
		for (int e = 0; e < 32; ++e) state[e] = 0.f;
		if (q < 2)
		{
			if (init)
			{
				const float4* ip = reinterpret_cast<const float4*>(init + (bh * 64 + r) * 64 + half * 32);
#pragma unroll
				for (int v = 0; v < 8; ++v)
				{
					const float4 t = ip[v];
					state[4 * v] = t.x; state[4 * v + 1] = t.y; state[4 * v + 2] = t.z; state[4 * v + 3] = t.w;
				}
			}
			uint8_t* prow = gen + OFF_P + r * 128;
#pragma unroll
			for (int v = 0; v < 4; ++v) *reinterpret_cast<Half8*>(prow + (((half * 4 + v) ^ (r & 7)) << 4)) = pack8(state + v * 8);
		}

		for (int j = 0; j < nsub; ++j)
		{
			const uint32_t par = static_cast<uint32_t>(j) & 1u;
			const int sbuf = j & 1;
			// ---- scalars of this block (two sets: a warp still in the previous block's epilogue reads the other one) --------
			if (warp < 4)
			{
				const float a2 = nx_dA * kLog2e;
				sc_dA2[sbuf][r] = a2;
				sc_q2[sbuf][r] = a2 - __log2f(nx_dt);
				// column factor of the pieces of S that lie below the diagonal piece of their rows: for l past the end e of the
				// 32-column piece that holds s, exp(dA[l] - dA[s]) dt[s] = exp(dA[l] - dA[e]) * (exp(dA[e] - dA[s]) dt[s]), both exponents <= 0
				sc_cf[sbuf][r] = ex2f(__shfl_sync(0xffffffffu, a2, 31) - a2) * nx_dt;
				sc_rowdec[sbuf][r] = ex2f((nx_dA - nx_base) * kLog2e);
				sc_w[sbuf][r] = ex2f((nx_last - nx_dA) * kLog2e) * nx_dt;
				if (r == QI - 1) sc_dec[sbuf] = ex2f((nx_dA - nx_base) * kLog2e);
			}
			named_barrier_sync(1, NCW * 32);
			const float dl2 = sc_dA2[sbuf][r];
			fetch_scalars(j + 1);

			// ---- S tiles from CB; B rows scaled in place ---------------------------------------------------------------------
			if (!dead && mbar_wait(cbb, par, abortp))
			{
				tc_fence_after();
				const int wrow0 = q * 32;
				uint8_t* srow = gen + OFF_S + (q >> 1) * TILE + r * 128;  // the diagonal piece of quadrant q lies in K-block q / 2
				// One 32 x 32 piece of S: thread = row r, columns s0 .. s0+31, weight = 2^(dl2 - q2[s]) with
				// q2[s] = dA[s] log2(e) - log2(dt[s]) (dt[s] = 0 gives q2 = +inf and the weight 0). DIAG: the piece holds the diagonal
				// (s0 == first row of the warp): causal mask, and D added on the diagonal.
				auto s_piece_exact = [&](const uint32_t* cbv, int s0, int ch, auto diag_tag) {
					constexpr bool DIAG = decltype(diag_tag)::value;
					const float4* qp = reinterpret_cast<const float4*>(sc_q2[sbuf] + s0);
#pragma unroll
					for (int v = 0; v < 4; ++v)
					{
						float o[8];
#pragma unroll
						for (int hq = 0; hq < 2; ++hq)
						{
							const float4 qv = qp[v * 2 + hq];
							const float qa[4] = { qv.x, qv.y, qv.z, qv.w };
#pragma unroll
							for (int e = 0; e < 4; ++e)
							{
								const int jj = v * 8 + hq * 4 + e;
								float val = __uint_as_float(cbv[jj]) * ex2f(dl2 - qa[e]);
								if (DIAG)
								{
									val = jj <= lane ? val : 0.f;
									if (jj == lane) val += dh;
								}
								o[hq * 4 + e] = val;
							}
						}
						*reinterpret_cast<Half8*>(srow + (((ch * 4 + v) ^ (r & 7)) << 4)) = pack8(o);
					}
				};
				// Pieces of 32 x 32 (rows of quadrant q, columns 32 pc .. 32 pc + 31, pc <= q); pc == q holds the diagonal. Dealt to the
				// two warps of a quadrant so that no warp has more than a diagonal piece and one other.
				auto s_piece_below = [&](int pc) {
					uint32_t cbv[32];
					tmem_ld_32x32(t_lane + static_cast<uint32_t>(pc * 32), cbv);
					const float rk = ex2f(dl2 - sc_dA2[sbuf][pc * 32 + 31]);
					const float4* cfp = reinterpret_cast<const float4*>(sc_cf[sbuf] + pc * 32);
					uint8_t* sr = gen + OFF_S + (pc >> 1) * TILE + r * 128;
					tmem_ld_wait();
#pragma unroll
					for (int v = 0; v < 4; ++v)
					{
						float o[8];
#pragma unroll
						for (int hq = 0; hq < 2; ++hq)
						{
							const float4 cf = cfp[v * 2 + hq];
							const float cfa[4] = { cf.x, cf.y, cf.z, cf.w };
#pragma unroll
							for (int e = 0; e < 4; ++e) o[hq * 4 + e] = __uint_as_float(cbv[v * 8 + hq * 4 + e]) * (rk * cfa[e]);
						}
						*reinterpret_cast<Half8*>(sr + ((((pc & 1) * 4 + v) ^ (r & 7)) << 4)) = pack8(o);
					}
				};
				auto s_piece_diag = [&]() {
					uint32_t cbv[32];
					tmem_ld_32x32(t_lane + static_cast<uint32_t>(wrow0), cbv);
					tmem_ld_wait();
					s_piece_exact(cbv, wrow0, q & 1, std::true_type{});
				};
				(void)srow;
				if (half == 0)
				{
					if (q < 2) s_piece_diag();                           // q0: its only piece; q1: the diagonal one
					else { s_piece_below(0); s_piece_below(1); }         // q2, q3: two pieces below
				}
				else
				{
					if (q == 1) s_piece_below(0);
					else if (q == 2) s_piece_diag();
					else if (q == 3) { s_piece_diag(); s_piece_below(2); }
				}
				// B[l, :] *= w[l] (a row-wise scale keeps every element where the swizzle put it). 1024 16-byte pieces: 20 per thread
				// for the warp without S work, 12 per thread for the warp with one piece below the diagonal.
				{
					int first = -1, count = 0;
					if (warp == 4) { first = lane; count = 20; }
					else if (warp == 5) { first = 640 + lane; count = 12; }
					for (int i = 0; i < count; ++i)
					{
						const int idx = first + i * 32;
						Half8* p = reinterpret_cast<Half8*>(gen + OFF_B + idx * 16);
						float f[8];
						unpack8(*p, f);
						const float sc = sc_w[sbuf][idx >> 3];
#pragma unroll
						for (int e = 0; e < 8; ++e) f[e] *= sc;
						*p = pack8(f);
					}
				}
			}
			else
				dead = true;
			fence_proxy_async_smem();
			tc_fence_before();
			__syncwarp();
			if (lane == 0) mbar_arrive(sb);

			// ---- y = Y + rowdec * Z (the state MMAs still run) ----------------------------------------------------------------
			if (!dead && mbar_wait(yb, par, abortp))
			{
				tc_fence_after();
				const float rd = sc_rowdec[sbuf][r];
				uint8_t* yrow = gen + OFF_Y + r * 128;
				// packed batch, last block of a sequence that does not fill it: the rows of this sequence go from registers to global
				// memory (64 contiguous bytes per thread), the rest of the tile belongs to the next sequence and is not written
				const bool ragged = VARLEN && (j + 1) * QI > len;
				__half* grow = VARLEN ? yv + (static_cast<int64_t>(tok0) + j * QI + r) * ys + h * 64 + half * 32 : nullptr;
				const bool grow_ok = VARLEN && j * QI + r < len;
#pragma unroll
				for (int hh = 0; hh < 2; ++hh)  // 16 columns at a time: fewer live registers
				{
					uint32_t yr[16], zr[16];
					tmem_ld_32x16(t_lane + 128u + static_cast<uint32_t>(half * 32 + hh * 16), yr);
					tmem_ld_32x16(t_lane + 192u + static_cast<uint32_t>(half * 32 + hh * 16), zr);
					tmem_ld_wait();
#pragma unroll
					for (int v = 0; v < 2; ++v)
					{
						float o[8];
#pragma unroll
						for (int e = 0; e < 8; ++e) o[e] = fmaf(rd, __uint_as_float(zr[v * 8 + e]), __uint_as_float(yr[v * 8 + e]));
						if (!ragged) *reinterpret_cast<Half8*>(yrow + (((half * 4 + hh * 2 + v) ^ (r & 7)) << 4)) = pack8(o);
						else if (grow_ok) *reinterpret_cast<Half8*>(grow + hh * 16 + v * 8) = pack8(o);
					}
				}
			}
			else
				dead = true;
			// ---- state <- decay * state + ST; its f16 copy is the next block's prev operand -------------------------------------
			if (q < 2)
			{
				if (!dead && mbar_wait(stb, par, abortp))
				{
					tc_fence_after();
					uint32_t sv[32];
					tmem_ld_32x32(t_lane + static_cast<uint32_t>(half * 32), sv);
					tmem_ld_wait();
					const float dec = sc_dec[sbuf];
#pragma unroll
					for (int e = 0; e < 32; ++e) state[e] = fmaf(dec, state[e], __uint_as_float(sv[e]));
					uint8_t* prow = gen + OFF_P + r * 128;
#pragma unroll
					for (int v = 0; v < 4; ++v) *reinterpret_cast<Half8*>(prow + (((half * 4 + v) ^ (r & 7)) << 4)) = pack8(state + v * 8);
				}
				else
					dead = true;
			}
			fence_proxy_async_smem();
			tc_fence_before();
			__syncwarp();
			if (lane == 0) mbar_arrive(epib);
		}
		if (dead && lane == 0) report_timeout(err_word, kErrScanWait);
		if (!dead && !*abortp && fin != nullptr && q < 2)
		{
			float4* fp = reinterpret_cast<float4*>(fin + (bh * 64 + r) * 64 + half * 32);
#pragma unroll
			for (int v = 0; v < 8; ++v) fp[v] = make_float4(state[4 * v], state[4 * v + 1], state[4 * v + 2], state[4 * v + 3]);
		}
	}

	__syncwarp();
	if (*abortp)
		for (int i = 0; i < 2000; ++i) __nanosleep(1000);  // loads that may still be in flight land before the CTA's memory is released
	tc_fence_before();
	__syncthreads();
	if (warp == 0)
	{
		tc_fence_after();
		tmem_dealloc(tmem_base, TMEM_COLS);
	}
}

// Shapes the one-kernel scan covers (the rest takes the staged kernels).
bool ssd_fused_supported(const SsdDims& d, const void* x, int64_t xs, const void* Bm, int64_t bs, const void* Cm, int64_t cs, const void* y,
	int64_t ys, const float* init, const float* fin)
{
	if (d.P != 64 || d.N != 64 || (d.Q != 128 && d.Q != 256)) return false;
	if (xs % 8 || bs % 8 || cs % 8 || ys % 8) return false;
	if (!aligned16(x) || !aligned16(Bm) || !aligned16(Cm) || !aligned16(y)) return false;
	if ((init && !aligned16(init)) || (fin && !aligned16(fin))) return false;
	if (d.batch > 0x7fffffffLL || d.seqlen > 0x7fffffffLL || d.batch * d.H > 0x7fffffffLL) return false;
	return true;
}

// 1: always, 0: never, -1: by size (environment variable B200_SSD_FUSED, read on every call so that a test can switch it)
static int fused_override()
{
	const char* e = std::getenv("B200_SSD_FUSED");
	if (!e || !*e) return -1;
	return e[0] == '0' ? 0 : 1;
}

// The one-kernel scan walks a sequence block by block (about 2.5 us per 128 tokens, whatever the number of (batch, head) pairs
// up to the 296 CTAs the GPU holds), the staged kernels spread the chunks of a sequence over the GPU: a few very long sequences
// are faster staged.
bool ssd_fused_preferred(const SsdDims& d)
{
	const int o = fused_override();
	if (o >= 0) return o == 1;
	const double waves = static_cast<double>(cdiv(d.batch * d.H, 2 * kNumSMs));
	const double nsub = static_cast<double>(d.nchunks) * (d.Q / sfused::QI);
	const double fused_us = waves * nsub * 2.6 + 8.0;
	const double staged_us = 35.0 + static_cast<double>(d.batch) * d.seqlen * d.H * 0.22e-3;
	return fused_us < staged_us;
}

int ssd_fused_tc(const __half* x, int64_t xs, const __half* Bm, int64_t bs, const __half* Cm, int64_t cs, const float* D,
	const float* init, __half* y, int64_t ys, float* fin, const SsdDims& d, const SsdWorkspace& w, cudaStream_t st)
{
	CUtensorMap tmX, tmB, tmC, tmY;
	const uint64_t L = static_cast<uint64_t>(d.seqlen), Bt = static_cast<uint64_t>(d.batch);
	int rc = tmap_3d_f16(&tmX, x, static_cast<uint64_t>(d.H) * 64, L, Bt, static_cast<uint64_t>(xs), L * xs, 64, sfused::QI);
	if (rc) return rc;
	rc = tmap_3d_f16(&tmB, Bm, static_cast<uint64_t>(d.G) * d.N, L, Bt, static_cast<uint64_t>(bs), L * bs, 64, sfused::QI);
	if (rc) return rc;
	rc = tmap_3d_f16(&tmC, Cm, static_cast<uint64_t>(d.G) * d.N, L, Bt, static_cast<uint64_t>(cs), L * cs, 64, sfused::QI);
	if (rc) return rc;
	rc = tmap_3d_f16(&tmY, y, static_cast<uint64_t>(d.H) * 64, L, Bt, static_cast<uint64_t>(ys), L * ys, 64, 64);
	if (rc) return rc;
	static bool smem_ok[64] = {};
	B200_CUDA_TRY(allow_dynamic_smem(ssd_fused_tc_kernel<false>, sfused::TOTAL, smem_ok));
	const unsigned grid = static_cast<unsigned>(d.batch * d.H);
	ssd_fused_tc_kernel<false><<<grid, sfused::THREADS, sfused::TOTAL, st>>>(tmX, tmB, tmC, tmY, D, w.dt, w.dacs, init, fin, d.seqlen, d.H,
		d.G, d.Q, d.nchunks, device_error_word(), nullptr, nullptr, 0, nullptr, 0);
	B200_LAUNCH_CHECK();
	return B200_OK;
}

// Packed batch: x / B / C / y are [total_tokens, features] tensors (row strides xs, bs, cs, ys), sequence s in rows cu[s] .. cu[s+1]-1;
// dt_rows / dacs_rows hold the dt stage's results per 128-token block of every sequence ([H][nblk][128], block coff[s] + j of
// sequence s); cu and coff are DEVICE arrays of nseq + 1 ints. init / fin: [nseq, H, P, N] fp32 or null.
bool ssd_fused_varlen_supported(int64_t total_tokens, int64_t nseq, int H, int P, int G, int N, const void* x, int64_t xs, const void* Bm,
	int64_t bs, const void* Cm, int64_t cs, const void* y, int64_t ys, const float* init, const float* fin)
{
	if (fused_override() == 0) return false;  // B200_SSD_FUSED=0 keeps every caller off the one-kernel scan, this one included
	if (P != 64 || N != 64 || H % G != 0) return false;
	if (xs % 8 || bs % 8 || cs % 8 || ys % 8) return false;
	if (!aligned16(x) || !aligned16(Bm) || !aligned16(Cm) || !aligned16(y)) return false;
	if ((init && !aligned16(init)) || (fin && !aligned16(fin))) return false;
	return total_tokens > 0 && total_tokens <= 0x7fffffffLL && nseq > 0 && nseq * H <= 0x7fffffffLL;
}

int ssd_fused_varlen_tc(const __half* x, int64_t xs, const __half* Bm, int64_t bs, const __half* Cm, int64_t cs, const float* D,
	const float* init, __half* y, int64_t ys, float* fin, int64_t total_tokens, int64_t nseq, int H, int G, const float* dt_rows,
	const float* dacs_rows, const int* cu, const int* coff, int nblk, cudaStream_t st)
{
	CUtensorMap tmX, tmB, tmC, tmY;
	const uint64_t L = static_cast<uint64_t>(total_tokens);
	int rc = tmap_3d_f16(&tmX, x, static_cast<uint64_t>(H) * 64, L, 1, static_cast<uint64_t>(xs), L * xs, 64, sfused::QI);
	if (rc) return rc;
	rc = tmap_3d_f16(&tmB, Bm, static_cast<uint64_t>(G) * 64, L, 1, static_cast<uint64_t>(bs), L * bs, 64, sfused::QI);
	if (rc) return rc;
	rc = tmap_3d_f16(&tmC, Cm, static_cast<uint64_t>(G) * 64, L, 1, static_cast<uint64_t>(cs), L * cs, 64, sfused::QI);
	if (rc) return rc;
	rc = tmap_3d_f16(&tmY, y, static_cast<uint64_t>(H) * 64, L, 1, static_cast<uint64_t>(ys), L * ys, 64, 64);
	if (rc) return rc;
	static bool smem_ok[64] = {};
	B200_CUDA_TRY(allow_dynamic_smem(ssd_fused_tc_kernel<true>, sfused::TOTAL, smem_ok));
	const unsigned grid = static_cast<unsigned>(nseq * H);
	ssd_fused_tc_kernel<true><<<grid, sfused::THREADS, sfused::TOTAL, st>>>(tmX, tmB, tmC, tmY, D, dt_rows, dacs_rows, init, fin, total_tokens, H,
		G, sfused::QI, 0, device_error_word(), cu, coff, nblk, y, ys);
	B200_LAUNCH_CHECK();
	return B200_OK;
}

}  // namespace b200
