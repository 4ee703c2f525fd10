// Y[M,N] = X[M,K] . W for the in_proj / out_proj of the Mamba2 mixer.
//
// f16: persistent, warp-specialised tcgen05 kernels. Large problems run on CTA pairs (cta_group::2, 256x256 tiles, see
// gemm_f16_tcgen05_pair_kernel); mid-size ones on one CTA per SM walking 128x256 output tiles; skinny ones (decode) on
// 128x64 tiles with a deep ring so that enough weight bytes are in flight to stream W at HBM rate. Roles per CTA:
//   warp 0    : TMA producer  - 128B-swizzled [128x64] X tiles and [256x64] W tiles into a 4-stage shared-memory ring
//   warp 1    : MMA issuer    - tcgen05.mma (M128 N256 K16, f16 in, fp32 accumulate) into one of two TMEM accumulators
//   warps 2-5 : epilogue      - tcgen05.ld the finished accumulator, round to f16, stage 32x64 sub-tiles in shared memory and
//                               write them with TMA stores (full 128-byte lines); overlaps the next tile's MMAs
// W is consumed as stored: (in,out) row-major tiles are fed MN-major, (out,in) row-major tiles K-major. Tails in M, N
// and K come from TMA zero fill and predicated stores. Every mbarrier wait is bounded.
//
// f32: exact fp32 SIMT kernel (64x64 tiles through shared memory), for Tensor<float32> callers.
#include "tcgen05.cuh"

namespace b200 {

// ---- f16 tcgen05 kernel -----------------------------------------------------------------------------------

namespace gemm {
constexpr int BM = 128, BK = 64;
constexpr int STG_BYTES = 32 * 128;      // per-warp output staging tile: 32 rows x 64 f16, 128B-swizzled
constexpr int THREADS = 192;

// Two tile shapes: 128x256 (one CTA per SM) for large problems, 128x64 (two CTAs per SM, all CTAs resident at once)
// for skinny ones such as the decode projections, where the job is to stream W once at full HBM bandwidth.
// A_ROWS: rows of X fetched per stage. With M <= 64 only 64 rows are loaded; the MMA still reads 128 rows of shared memory
// (the second half is whatever follows in the ring) and the accumulator rows it produces from them are never stored.
template <int BN_, int STAGES_, int STG_BUFS_, int MIN_CTAS_, int A_ROWS_ = 128>
struct Cfg
{
	static constexpr int BN = BN_, STAGES = STAGES_, STG_BUFS = STG_BUFS_, MIN_CTAS = MIN_CTAS_, A_ROWS = A_ROWS_;
	static constexpr int A_BYTES = A_ROWS * BK * 2;
	static constexpr int B_BYTES = BN * BK * 2;
	static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
	static constexpr int STG_TOTAL = 4 * STG_BUFS * STG_BYTES;
	static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + STG_TOTAL + 1024;  // + slack to align the ring to 1024 B
	static constexpr uint32_t TMEM_COLS = 2 * BN;  // two fp32 accumulators
};
using CfgWide = Cfg<256, 4, 2, 1>;
using CfgSkinny = Cfg<64, 8, 1, 1>;        // 8 x 24 KiB ring
using CfgSkinny64 = Cfg<64, 13, 1, 1, 64>;  // M <= 64: 13 x 16 KiB ring, 104 KiB of W in flight per SM
}  // namespace gemm

template <int B_MN, class C>
__global__ void __launch_bounds__(gemm::THREADS, C::MIN_CTAS) gemm_f16_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA,
	const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmY, int M, int N, int K, int m_tiles, int n_tiles,
	uint32_t* err_word, const __half* __restrict__ residual, int64_t ldr,
	uint32_t spin_limit /* polls after which a wait gives up */, int producer_short /* K-blocks per tile that the producer leaves out: 0
	except in the self-test of the give-up path, where the MMA thread then waits for a stage that never fills */)
{
	using namespace gemm;
	using namespace tc;
	constexpr int BN = C::BN, STAGES = C::STAGES, STAGE_BYTES = C::STAGE_BYTES, STG_BUFS = C::STG_BUFS, A_BYTES = C::A_BYTES;
	constexpr uint32_t TMEM_COLS = C::TMEM_COLS;
	extern __shared__ uint8_t smem_raw[];
	__shared__ uint64_t bar_full[STAGES], bar_empty[STAGES], bar_tfull[2], bar_tempty[2];
	__shared__ uint32_t tmem_slot;
	__shared__ int abort_flag;

	const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
	const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
	const int k_blocks = (K + BK - 1) / BK;
	const int num_tiles = m_tiles * n_tiles;
	volatile int* abortp = &abort_flag;

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
			mbar_init(smem_u32(&bar_tempty[a]), 4);
		}
		fence_mbar_init();
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
			prefetch_tmap(&tmA);
			prefetch_tmap(&tmB);
			int stage = 0;
			uint32_t phase = 0;
			for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x)
			{
				const int m0 = (tile % m_tiles) * BM;
				const int n0 = (tile / m_tiles) * BN;
				for (int kb = 0; kb < k_blocks - producer_short; ++kb)
				{
					if (!mbar_wait(smem_u32(&bar_empty[stage]), phase ^ 1u, abortp, spin_limit))
					{
						report_timeout(err_word, kErrProducerWait);
						goto role_done;
					}
					const uint32_t full = smem_u32(&bar_full[stage]);
					const uint32_t a_s = ring + stage * STAGE_BYTES;
					const uint32_t b_s = a_s + A_BYTES;
					mbar_arrive_expect_tx(full, STAGE_BYTES);
					tma_load_2d(a_s, &tmA, full, kb * BK, m0);
					if (B_MN == 0)
					{
						tma_load_2d(b_s, &tmB, full, kb * BK, n0);  // W^T [N,K]: one [BN n x 64 k] box
					}
					else
					{
#pragma unroll
						for (int j = 0; j < BN / 64; ++j)  // W [K,N]: BN/64 boxes of [64 k x 64 n]
							tma_load_2d(b_s + j * (BK * 128), &tmB, full, n0 + j * 64, kb * BK);
					}
					if (++stage == STAGES) { stage = 0; phase ^= 1u; }
				}
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
			for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x)
			{
				if (!mbar_wait(smem_u32(&bar_tempty[acc]), acc_phase ^ 1u, abortp, spin_limit))
				{
					report_timeout(err_word, kErrMmaWaitTmem);
					goto role_done;
				}
				tc_fence_after();
				const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
				for (int kb = 0; kb < k_blocks; ++kb)
				{
					if (!mbar_wait(smem_u32(&bar_full[stage]), phase, abortp, spin_limit))
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
						// K-major: 16 f16 = 32 B along the swizzled row; MN-major: 16 k-rows = two 1024-byte groups
						const uint64_t a_k = a_desc + static_cast<uint64_t>(k * 2);
						const uint64_t b_k = b_desc + static_cast<uint64_t>(B_MN ? k * 128 : k * 2);
						mma_f16_ss(d_tmem, a_k, b_k, idesc, (kb | k) != 0 ? 1u : 0u);
					}
					mma_commit(smem_u32(&bar_empty[stage]));  // frees the stage once these MMAs have read it
					if (++stage == STAGES) { stage = 0; phase ^= 1u; }
				}
				mma_commit(smem_u32(&bar_tfull[acc]));  // accumulator complete
				if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
			}
		}
	}
	else
	{
		const int q = warp & 3;  // TMEM lane quadrant this warp may read
		uint8_t* stg = smem_raw + (ring - smem_u32(smem_raw)) + STAGES * STAGE_BYTES + q * (STG_BUFS * STG_BYTES);
		const uint32_t stg_s = ring + STAGES * STAGE_BYTES + q * (STG_BUFS * STG_BYTES);
		if (lane == 0) prefetch_tmap(&tmY);
		int acc = 0;
		uint32_t acc_phase = 0;
		uint32_t nchunk = 0;
		for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x)
		{
			const int m0 = (tile % m_tiles) * BM;
			const int n0 = (tile / m_tiles) * BN;
			if (!mbar_wait(smem_u32(&bar_tfull[acc]), acc_phase, abortp, spin_limit))
			{
				if (lane == 0) report_timeout(err_word, kErrEpilogueWait);
				goto role_done;
			}
			tc_fence_after();
			const uint32_t t_base = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(acc * BN);
#pragma unroll 1
			for (int c = 0; c < BN / 64; ++c)
			{
				if (n0 + c * 64 >= N) break;  // warp-uniform
				uint32_t r0[32], r1[32];
				tmem_ld_32x32(t_base + static_cast<uint32_t>(c * 64), r0);
				tmem_ld_32x32(t_base + static_cast<uint32_t>(c * 64 + 32), r1);
				// the staging buffer about to be rewritten must have been read by its store
				if (lane == 0) bulk_wait_group_read<STG_BUFS - 1>();
				__syncwarp();
				tmem_ld_wait();
				const uint32_t buf = nchunk % STG_BUFS;
				uint8_t* srow = stg + buf * STG_BYTES + lane * 128;
				// optional residual: Y = X.W + R (R f16, row stride ldr), added in fp32 before the one rounding
				const int rrow = m0 + q * 32 + lane;
				const __half* rp = residual != nullptr && rrow < M ? residual + static_cast<int64_t>(rrow) * ldr + n0 + c * 64 : nullptr;
#pragma unroll
				for (int v = 0; v < 8; ++v)
				{
					const uint32_t* src = v < 4 ? r0 + v * 8 : r1 + (v - 4) * 8;
					float f[8];
#pragma unroll
					for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(src[e]);
					if (rp != nullptr && n0 + c * 64 + v * 8 < N)  // N % 8 == 0
					{
						float rv[8];
						unpack8(*reinterpret_cast<const Half8*>(rp + v * 8), rv);
#pragma unroll
						for (int e = 0; e < 8; ++e) f[e] += rv[e];
					}
					*reinterpret_cast<Half8*>(srow + ((v ^ (lane & 7)) << 4)) = pack8(f);
				}
				fence_proxy_async_smem();
				__syncwarp();
				if (lane == 0)
				{
					tma_store_2d(&tmY, stg_s + buf * STG_BYTES, n0 + c * 64, m0 + q * 32);  // clipped at M and N
					bulk_commit_group();
				}
				++nchunk;
			}
			tc_fence_before();
			__syncwarp();
			if (lane == 0) mbar_arrive(smem_u32(&bar_tempty[acc]));
			if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
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

// ---- CTA-pair variant (cta_group::2) ---------------------------------------------------------------------------------
// Two CTAs of a cluster own one 256x256 output tile: each loads its 128 rows of X and HALF of the W tile (128 of the 256
// output columns), the leader CTA issues tcgen05.mma.cta_group::2 (M = 256), which reads both CTAs' shared memory, and
// each CTA's TMEM receives its 128 rows x 256 columns. Per output tile the pair fetches half the W bytes that two
// independent CTAs would, which lifts the L2 -> shared-memory bound of the single-CTA kernel. No load is multicast.
namespace gemm2 {
constexpr int BM = 128, BN = 256, BK = 64, STAGES = 6;
constexpr int A_BYTES = BM * BK * 2;        // this CTA's rows of X: 16 KiB
constexpr int B_BYTES = (BN / 2) * BK * 2;  // this CTA's half of the W tile: 16 KiB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int STG_BYTES = 32 * 128;
constexpr int STG_BUFS = 2;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 4 * STG_BUFS * STG_BYTES + 1024;
constexpr int THREADS = 192;
constexpr uint32_t TMEM_COLS = 512;
}  // namespace gemm2

// Tile order of the pair kernel. panel = 0: down the rows of X first (tile t -> row block t % m_tiles, column block t / m_tiles).
// panel = G > 0: the column blocks of W in panels of G; inside a panel across its columns first, then to the next row block, the
// row blocks taken from the last to the first. A wave of 74 tiles then touches 74 / G row blocks of X and G column blocks of W.
__device__ __forceinline__ void pair_tile_coords(int tile, int m_tiles, int n_tiles, int panel, int* tm, int* tn)
{
	if (panel == 0)
	{
		*tm = tile % m_tiles;
		*tn = tile / m_tiles;
		return;
	}
	const int per_panel = panel * m_tiles;
	const int p = tile / per_panel;
	const int r = tile - p * per_panel;
	const int width = min(panel, n_tiles - p * panel);  // the last panel may be narrower
	*tm = m_tiles - 1 - r / width;
	*tn = p * panel + r % width;
}

template <int B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(gemm2::THREADS, 1) gemm_f16_tcgen05_pair_kernel(
	const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmY, int M,
	int N, int K, int m_tiles /* of 256 rows */, int n_tiles, uint32_t* err_word, const __half* __restrict__ residual, int64_t ldr,
	int panel /* tile order, see pair_tile_coords */)
{
	using namespace gemm2;
	using namespace tc;
	extern __shared__ uint8_t smem_raw[];
	__shared__ uint64_t bar_full[STAGES], bar_empty[STAGES], bar_tfull[2], bar_tempty[2];
	__shared__ uint32_t tmem_slot;
	__shared__ int abort_flag;

	const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
	const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
	const uint32_t rank = cluster_ctarank();  // 0 = leader
	const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
	const int k_blocks = (K + BK - 1) / BK;
	const int num_tiles = m_tiles * n_tiles;
	volatile int* abortp = &abort_flag;

	if (threadIdx.x == 0)
	{
		abort_flag = 0;
		for (int s = 0; s < STAGES; ++s)
		{
			mbar_init(smem_u32(&bar_full[s]), 1);   // used in the leader only: its own arrive.expect_tx covers both CTAs' bytes
			mbar_init(smem_u32(&bar_empty[s]), 1);  // one pair-wide commit per use
		}
		for (int a = 0; a < 2; ++a)
		{
			mbar_init(smem_u32(&bar_tfull[a]), 1);
			mbar_init(smem_u32(&bar_tempty[a]), 8);  // leader only: 4 epilogue warps of each CTA
		}
		fence_mbar_init();
	}
	if (warp == 1)
	{
		tmem_alloc_pair(smem_u32(&tmem_slot), TMEM_COLS);
		tmem_relinquish_pair();
	}
	tc_fence_before();
	__syncthreads();
	cluster_sync();  // the peer's barriers exist before anything is signalled across CTAs
	tc_fence_after();
	const uint32_t tmem_base = tmem_slot;

	if (warp == 0)
	{
		if (lane == 0)
		{
			prefetch_tmap(&tmA);
			prefetch_tmap(&tmB);
			int stage = 0;
			uint32_t phase = 0;
			for (int tile = pair; tile < num_tiles; tile += npairs)
			{
				int tm, tn;
				pair_tile_coords(tile, m_tiles, n_tiles, panel, &tm, &tn);
				const int m0 = tm * (2 * BM) + static_cast<int>(rank) * BM;
				const int n0 = tn * BN + static_cast<int>(rank) * (BN / 2);
				for (int kb = 0; kb < k_blocks; ++kb)
				{
					if (!mbar_wait(smem_u32(&bar_empty[stage]), phase ^ 1u, abortp))
					{
						report_timeout(err_word, kErrProducerWait);
						goto role_done;
					}
					// completion bytes of BOTH CTAs are counted on the leader's barrier
					const uint32_t full = map_to_cta(smem_u32(&bar_full[stage]), 0);
					const uint32_t a_s = ring + stage * STAGE_BYTES;
					const uint32_t b_s = a_s + A_BYTES;
					if (rank == 0) mbar_arrive_expect_tx(smem_u32(&bar_full[stage]), 2 * STAGE_BYTES);
					tma_load_2d_pair(a_s, &tmA, full, kb * BK, m0);
					if (B_MN == 0)
					{
						tma_load_2d_pair(b_s, &tmB, full, kb * BK, n0);  // W^T [N,K]: [128 n x 64 k]
					}
					else
					{
#pragma unroll
						for (int j = 0; j < BN / 2 / 64; ++j)  // W [K,N]: two boxes of [64 k x 64 n]
							tma_load_2d_pair(b_s + j * (BK * 128), &tmB, full, n0 + j * 64, kb * BK);
					}
					if (++stage == STAGES) { stage = 0; phase ^= 1u; }
				}
			}
		}
	}
	else if (warp == 1)
	{
		if (lane == 0 && rank == 0)
		{
			constexpr uint32_t idesc = make_idesc_f16(2 * BM, BN, B_MN);
			int stage = 0;
			uint32_t phase = 0;
			int acc = 0;
			uint32_t acc_phase = 0;
			for (int tile = pair; tile < num_tiles; tile += npairs)
			{
				if (!mbar_wait(smem_u32(&bar_tempty[acc]), acc_phase ^ 1u, abortp))
				{
					report_timeout(err_word, kErrMmaWaitTmem);
					goto role_done;
				}
				tc_fence_after();
				const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
				for (int kb = 0; kb < k_blocks; ++kb)
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
						mma_f16_ss_pair(d_tmem, a_k, b_k, idesc, (kb | k) != 0 ? 1u : 0u);
					}
					mma_commit_pair(smem_u32(&bar_empty[stage]), 3);  // frees the stage in both CTAs
					if (++stage == STAGES) { stage = 0; phase ^= 1u; }
				}
				mma_commit_pair(smem_u32(&bar_tfull[acc]), 3);  // accumulators complete in both CTAs
				if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
			}
		}
	}
	else
	{
		const int q = warp & 3;
		uint8_t* stg = smem_raw + (ring - smem_u32(smem_raw)) + STAGES * STAGE_BYTES + q * (STG_BUFS * STG_BYTES);
		const uint32_t stg_s = ring + STAGES * STAGE_BYTES + q * (STG_BUFS * STG_BYTES);
		if (lane == 0) prefetch_tmap(&tmY);
		int acc = 0;
		uint32_t acc_phase = 0;
		uint32_t nchunk = 0;
		for (int tile = pair; tile < num_tiles; tile += npairs)
		{
			int tm, tn;
			pair_tile_coords(tile, m_tiles, n_tiles, panel, &tm, &tn);
			const int m0 = tm * (2 * BM) + static_cast<int>(rank) * BM;
			const int n0 = tn * BN;
			if (!mbar_wait(smem_u32(&bar_tfull[acc]), acc_phase, abortp))
			{
				if (lane == 0) report_timeout(err_word, kErrEpilogueWait);
				goto role_done;
			}
			tc_fence_after();
			const uint32_t t_base = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(acc * BN);
#pragma unroll 1
			for (int c = 0; c < BN / 64; ++c)
			{
				if (n0 + c * 64 >= N) break;  // warp-uniform
				uint32_t r0[32], r1[32];
				tmem_ld_32x32(t_base + static_cast<uint32_t>(c * 64), r0);
				tmem_ld_32x32(t_base + static_cast<uint32_t>(c * 64 + 32), r1);
				if (lane == 0) bulk_wait_group_read<STG_BUFS - 1>();
				__syncwarp();
				tmem_ld_wait();
				const uint32_t buf = nchunk % STG_BUFS;
				uint8_t* srow = stg + buf * STG_BYTES + lane * 128;
				// optional residual: Y = X.W + R (R f16, row stride ldr), added in fp32 before the one rounding
				const int rrow = m0 + q * 32 + lane;
				const __half* rp = residual != nullptr && rrow < M ? residual + static_cast<int64_t>(rrow) * ldr + n0 + c * 64 : nullptr;
#pragma unroll
				for (int v = 0; v < 8; ++v)
				{
					const uint32_t* src = v < 4 ? r0 + v * 8 : r1 + (v - 4) * 8;
					float f[8];
#pragma unroll
					for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(src[e]);
					if (rp != nullptr && n0 + c * 64 + v * 8 < N)  // N % 8 == 0
					{
						float rv[8];
						unpack8(*reinterpret_cast<const Half8*>(rp + v * 8), rv);
#pragma unroll
						for (int e = 0; e < 8; ++e) f[e] += rv[e];
					}
					*reinterpret_cast<Half8*>(srow + ((v ^ (lane & 7)) << 4)) = pack8(f);
				}
				fence_proxy_async_smem();
				__syncwarp();
				if (lane == 0)
				{
					tma_store_2d(&tmY, stg_s + buf * STG_BYTES, n0 + c * 64, m0 + q * 32);
					bulk_commit_group();
				}
				++nchunk;
			}
			tc_fence_before();
			__syncwarp();
			if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&bar_tempty[acc]), 0));  // the leader's MMA thread waits on it
			if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
		}
		if (lane == 0) bulk_wait_group<0>();
	}

role_done:
	__syncwarp();
	if (*abortp)
		for (int i = 0; i < 2000; ++i) __nanosleep(1000);
	tc_fence_before();
	__syncthreads();
	cluster_sync();  // neither CTA releases shared or tensor memory while the peer may still touch it
	if (warp == 1)
	{
		tc_fence_after();
		tmem_dealloc_pair(tmem_base, TMEM_COLS);
	}
}

template <int B_MN>
static int launch_gemm_pair(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmY, int M, int N, int K, cudaStream_t st,
	const __half* residual, int64_t ldr)
{
	using namespace gemm2;
	static bool smem_ok[64] = {};
	B200_CUDA_TRY(allow_dynamic_smem(gemm_f16_tcgen05_pair_kernel<B_MN>, SMEM_BYTES, smem_ok));
	const int m_tiles = static_cast<int>(cdiv(M, 2 * BM)), n_tiles = static_cast<int>(cdiv(N, BN));
	const int64_t tiles = static_cast<int64_t>(m_tiles) * n_tiles;
	const int64_t pairs = tiles < kNumSMs / 2 ? tiles : kNumSMs / 2;
	// Tile order (pair_tile_coords). The pairs of one wave work on consecutive tiles; what every wave touches has to stay in L2
	// between waves, and what a CTA finds there is about half of the 126 MB (each die keeps its own copy of lines both use). Dealt
	// down the rows first, a wave touches every row block of X: fine while X fits (in_proj at 8192 tokens, X 34 MB: ncu counted
	// 83 MB read from DRAM per launch against 68 MB of operands), not beyond (out_proj there, X 67 MB and W 17 MB: 206 MB against
	// 84 MB). A larger X is walked in panels of column blocks whose slab of W (~30 MB) stays resident while the row blocks stream
	// past it once per panel, from the last row block to the first (whatever produced X most likely wrote its rows in ascending
	// order, so the last ones are the ones still in L2). Measured: 8192 tokens, out_proj 107.1 -> 105.5 us; 16384 tokens of the
	// 7B-shaped layer (X 117 / 235 MB), panels of 16 / 8 against one panel of all columns: in_proj 1.416 -> 1.257 ms, out_proj
	// 0.654 -> 0.618 ms, step 2.60 -> 2.37 ms; panels at 8192 tokens for in_proj as well: 0.4400 -> 0.4432 ms per step.
	const double x_bytes = 2.0 * M * K;
	int panel = 0;
	if (x_bytes > 48e6)
	{
		panel = static_cast<int>(30e6 / (512.0 * K));
		panel = panel < 4 ? 4 : panel;
		panel = panel > n_tiles ? n_tiles : panel;
	}
	gemm_f16_tcgen05_pair_kernel<B_MN><<<static_cast<unsigned>(2 * pairs), THREADS, SMEM_BYTES, st>>>(tmA, tmB, tmY, M, N, K, m_tiles,
		n_tiles, device_error_word(), residual, ldr, panel);
	B200_LAUNCH_CHECK();
	return B200_OK;
}

// What the self-test of the give-up path asks of the next launch of the single-CTA kernel (b200_debug_linear_starved_producer).
struct GemmDebug
{
	uint32_t spin_limit = tc::kSpinLimit;
	int producer_short = 0;
};

template <int B_MN, class C>
static int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmY, int M, int N, int K, cudaStream_t st,
	const __half* residual, int64_t ldr, const GemmDebug& dbg = GemmDebug())
{
	using namespace gemm;
	static bool smem_ok[64] = {};
	B200_CUDA_TRY(allow_dynamic_smem(gemm_f16_tcgen05_kernel<B_MN, C>, C::SMEM_BYTES, smem_ok));
	const int m_tiles = static_cast<int>(cdiv(M, BM)), n_tiles = static_cast<int>(cdiv(N, C::BN));
	const int64_t tiles = static_cast<int64_t>(m_tiles) * n_tiles;
	const int64_t slots = static_cast<int64_t>(kNumSMs) * C::MIN_CTAS;
	const unsigned grid = static_cast<unsigned>(tiles < slots ? tiles : slots);
	gemm_f16_tcgen05_kernel<B_MN, C><<<grid, THREADS, C::SMEM_BYTES, st>>>(tmA, tmB, tmY, M, N, K, m_tiles, n_tiles, device_error_word(),
		residual, ldr, dbg.spin_limit, dbg.producer_short);
	B200_LAUNCH_CHECK();
	return B200_OK;
}

// Which tensor-core kernel a problem takes: CTA pairs on 256x256 tiles once those fill half the machine, wide 128x256 tiles once
// they fill most of it, otherwise skinny 128x64 tiles (two CTAs per SM), with 64-row X boxes for M <= 64.
struct GemmChoice
{
	bool paired, wide, tiny_m;
};
static GemmChoice gemm_f16_choice(int64_t M, int64_t N)
{
	GemmChoice c;
	c.wide = cdiv(M, gemm::BM) * cdiv(N, 256) >= 96;
	c.paired = cdiv(M, 256) * cdiv(N, 256) >= kNumSMs / 2;
	c.tiny_m = !c.paired && !c.wide && M <= 64;
	return c;
}

// true when the tensor-core kernels can take the problem: TMA needs 16-byte aligned bases and row strides
static bool gemm_f16_tc_ok(const void* x, int64_t ldx, const void* w, const void* y, int64_t ldy, int64_t K, int64_t N)
{
	return K % 8 == 0 && N % 8 == 0 && ldx % 8 == 0 && ldy % 8 == 0 && aligned16(x) && aligned16(w) && aligned16(y);
}

static int gemm_f16(const __half* x, int64_t ldx, const __half* w, int w_layout, __half* y, int64_t ldy, int64_t M, int64_t K,
	int64_t N, cudaStream_t st, const __half* residual = nullptr, int64_t ldr = 0, const GemmDebug& dbg = GemmDebug())
{
	using namespace gemm;
	if (!gemm_f16_tc_ok(x, ldx, w, y, ldy, K, N)) return B200_ERR_MISALIGNED;
	if (residual && (ldr % 8 != 0 || !aligned16(residual))) return B200_ERR_MISALIGNED;
	if (M > 0x7fffffffLL || N > 0x7fffffffLL || K > 0x7fffffffLL) return B200_ERR_UNSUPPORTED;
	const GemmChoice ch = gemm_f16_choice(M, N);
	const bool wide = ch.wide, paired = ch.paired, tiny_m = ch.tiny_m;
	const uint32_t bn = paired ? 128 : (wide ? 256 : 64);
	CUtensorMap tmA, tmB, tmY;
	int rc = tmap_2d_f16(&tmY, y, static_cast<uint64_t>(M), static_cast<uint64_t>(N), static_cast<uint64_t>(ldy), 64, 32);
	if (rc) return rc;
	rc = tmap_2d_f16(&tmA, x, static_cast<uint64_t>(M), static_cast<uint64_t>(K), static_cast<uint64_t>(ldx), BK, tiny_m ? 64 : BM);
	if (rc) return rc;
	if (w_layout == B200_W_NK)
		rc = tmap_2d_f16(&tmB, w, static_cast<uint64_t>(N), static_cast<uint64_t>(K), static_cast<uint64_t>(K), BK, bn);
	else
		rc = tmap_2d_f16(&tmB, w, static_cast<uint64_t>(K), static_cast<uint64_t>(N), static_cast<uint64_t>(N), 64, BK);
	if (rc) return rc;
	const int m = static_cast<int>(M), n = static_cast<int>(N), k = static_cast<int>(K);
	if (paired) return w_layout == B200_W_NK ? launch_gemm_pair<0>(tmA, tmB, tmY, m, n, k, st, residual, ldr) : launch_gemm_pair<1>(tmA, tmB, tmY, m, n, k, st, residual, ldr);
	if (w_layout == B200_W_NK)
	{
		if (wide) return launch_gemm<0, CfgWide>(tmA, tmB, tmY, m, n, k, st, residual, ldr, dbg);
		return tiny_m ? launch_gemm<0, CfgSkinny64>(tmA, tmB, tmY, m, n, k, st, residual, ldr, dbg) : launch_gemm<0, CfgSkinny>(tmA, tmB, tmY, m, n, k, st, residual, ldr, dbg);
	}
	if (wide) return launch_gemm<1, CfgWide>(tmA, tmB, tmY, m, n, k, st, residual, ldr, dbg);
	return tiny_m ? launch_gemm<1, CfgSkinny64>(tmA, tmB, tmY, m, n, k, st, residual, ldr, dbg) : launch_gemm<1, CfgSkinny>(tmA, tmB, tmY, m, n, k, st, residual, ldr, dbg);
}

// Y = X . W + R, f16 (R: residual stream of the layer around the projection, added in the epilogue).
int linear_f16_residual(const void* x, int64_t ldx, const void* w, int w_layout, void* y, int64_t ldy, int64_t M, int64_t K, int64_t N,
	const void* residual, int64_t ldr, cudaStream_t st)
{
	if (w_layout != B200_W_KN && w_layout != B200_W_NK) return B200_ERR_UNSUPPORTED;
	if (M == 0 || N == 0) return B200_OK;
	return gemm_f16(static_cast<const __half*>(x), ldx, static_cast<const __half*>(w), w_layout, static_cast<__half*>(y), ldy, M, K, N, st,
		static_cast<const __half*>(residual), ldr);
}

// ---- SIMT kernel (fp32 tensors; f16 tensors whose shape or alignment the tensor-core kernels cannot take) -----------
// 64x64 output tile, 16x16 threads, 4x4 per thread, k in slices of 16, fp32 accumulation in the order k = 0, 1, 2, ...
// ws_k / ws_n: element strides of W along k and n.
template <typename T>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const T* __restrict__ X, int64_t ldx, const T* __restrict__ W,
	int64_t ws_k, int64_t ws_n, T* __restrict__ Y, int64_t ldy, int M, int N, int K)
{
	__shared__ __align__(16) float sa[16][64 + 4];  // [k][m]
	__shared__ __align__(16) float sb[16][64 + 4];  // [k][n]
	const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
	const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
	float acc[4][4] = {};
	for (int k0 = 0; k0 < K; k0 += 16)
	{
		for (int idx = threadIdx.x; idx < 16 * 64; idx += 256)
		{
			{
				const int kk = idx & 15, mm = idx >> 4;  // X: k contiguous
				const int m = m0 + mm, k = k0 + kk;
				sa[kk][mm] = (m < M && k < K) ? ldf(X + static_cast<int64_t>(m) * ldx + k) : 0.f;
			}
			{
				int kk, nn;
				if (ws_n == 1) { nn = idx & 63; kk = idx >> 6; }  // W (K,N): n contiguous
				else { kk = idx & 15; nn = idx >> 4; }             // W (N,K): k contiguous
				const int n = n0 + nn, k = k0 + kk;
				sb[kk][nn] = (n < N && k < K) ? ldf(W + static_cast<int64_t>(k) * ws_k + static_cast<int64_t>(n) * ws_n) : 0.f;
			}
		}
		__syncthreads();
#pragma unroll
		for (int kk = 0; kk < 16; ++kk)
		{
			const float4 a = *reinterpret_cast<const float4*>(&sa[kk][ty * 4]);
			const float4 b = *reinterpret_cast<const float4*>(&sb[kk][tx * 4]);
			const float ar[4] = { a.x, a.y, a.z, a.w };
			const float br[4] = { b.x, b.y, b.z, b.w };
#pragma unroll
			for (int i = 0; i < 4; ++i)
#pragma unroll
				for (int j = 0; j < 4; ++j) acc[i][j] += ar[i] * br[j];
		}
		__syncthreads();
	}
#pragma unroll
	for (int i = 0; i < 4; ++i)
#pragma unroll
		for (int j = 0; j < 4; ++j)
		{
			const int m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
			if (m < M && n < N) stf(Y + static_cast<int64_t>(m) * ldy + n, acc[i][j]);
		}
}

template <typename T>
static int gemm_simt(const T* x, int64_t ldx, const T* w, int w_layout, T* y, int64_t ldy, int64_t M, int64_t K, int64_t N,
	cudaStream_t st)
{
	if (M > 0x7fffffffLL || N > 0x7fffffffLL || K > 0x7fffffffLL) return B200_ERR_UNSUPPORTED;
	const dim3 g(static_cast<unsigned>(cdiv(N, 64)), static_cast<unsigned>(cdiv(M, 64)));
	if (g.y > 65535u) return B200_ERR_UNSUPPORTED;
	const int64_t ws_k = w_layout == B200_W_KN ? N : 1;
	const int64_t ws_n = w_layout == B200_W_KN ? 1 : K;
	gemm_simt_kernel<T><<<g, 256, 0, st>>>(x, ldx, w, ws_k, ws_n, y, ldy, static_cast<int>(M), static_cast<int>(N),
		static_cast<int>(K));
	B200_LAUNCH_CHECK();
	return B200_OK;
}

}  // namespace b200

using namespace b200;

extern "C" int b200_linear(int dtype, const void* x, int64_t ldx, const void* w, int w_layout, void* y, int64_t ldy,
	int64_t M, int64_t K, int64_t N, void* stream)
{
	if (!x || !w || !y) return B200_ERR_NULL;
	if (M < 0 || K <= 0 || N <= 0 || ldx < K || ldy < N) return B200_ERR_BAD_SHAPE;
	if (w_layout != B200_W_KN && w_layout != B200_W_NK) return B200_ERR_UNSUPPORTED;
	if (M == 0) return B200_OK;
	cudaStream_t st = static_cast<cudaStream_t>(stream);
	if (dtype == B200_F16)
	{
		// anyGPU's tensor_linear takes any shape: what TMA cannot address (a dimension or stride that is not a multiple of 8
		// elements, a base off a 16-byte boundary) runs on the SIMT kernel instead of being refused
		if (!gemm_f16_tc_ok(x, ldx, w, y, ldy, K, N))
			return gemm_simt<__half>(static_cast<const __half*>(x), ldx, static_cast<const __half*>(w), w_layout, static_cast<__half*>(y),
				ldy, M, K, N, st);
		return gemm_f16(static_cast<const __half*>(x), ldx, static_cast<const __half*>(w), w_layout, static_cast<__half*>(y), ldy, M,
			K, N, st);
	}
	if (dtype == B200_F32)
		return gemm_simt<float>(static_cast<const float*>(x), ldx, static_cast<const float*>(w), w_layout, static_cast<float*>(y), ldy, M,
			K, N, st);
	return B200_ERR_UNSUPPORTED;
}

extern "C" int b200_debug_linear_starved_producer(const void* x, int64_t ldx, const void* w, int w_layout, void* y, int64_t ldy, int64_t M,
	int64_t K, int64_t N, uint32_t spin_limit, void* stream)
{
	if (!x || !w || !y) return B200_ERR_NULL;
	if (M <= 0 || K < 2 * gemm::BK || N <= 0 || ldx < K || ldy < N || spin_limit == 0) return B200_ERR_BAD_SHAPE;
	if (w_layout != B200_W_KN && w_layout != B200_W_NK) return B200_ERR_UNSUPPORTED;
	if (!gemm_f16_tc_ok(x, ldx, w, y, ldy, K, N) || gemm_f16_choice(M, N).paired) return B200_ERR_UNSUPPORTED;  // single-CTA kernel only
	GemmDebug dbg;
	dbg.spin_limit = spin_limit;
	dbg.producer_short = 1;
	return gemm_f16(static_cast<const __half*>(x), ldx, static_cast<const __half*>(w), w_layout, static_cast<__half*>(y), ldy, M, K, N,
		static_cast<cudaStream_t>(stream), nullptr, 0, dbg);
}

extern "C" const char* b200_linear_kernel_name(int dtype, int64_t M, int64_t K, int64_t N)
{
	if (dtype == B200_F32) return "gemm_simt_kernel<float>";
	if (dtype != B200_F16 || M <= 0 || K <= 0 || N <= 0) return "";
	if (K % 8 != 0 || N % 8 != 0) return "gemm_simt_kernel<__half>";
	const GemmChoice c = gemm_f16_choice(M, N);
	if (c.paired) return "gemm_f16_tcgen05_pair_kernel";
	return c.wide ? "gemm_f16_tcgen05_kernel (128x256 tiles)" : (c.tiny_m ? "gemm_f16_tcgen05_kernel (64-row X, 128x64 tiles)" : "gemm_f16_tcgen05_kernel (128x64 tiles)");
}
