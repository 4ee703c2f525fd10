// Tensor-core (tcgen05 / TMEM / TMA) stages of the SSD chunked scan for f16 activations.
//
// chunk state  : states[(h,p), n] = sum_l (x[l,h,p] * exp(dAcs[last]-dAcs[l]) * dt[l]) * B[l,n]
//                one CTA per (batch, chunk, head pair): M = 2 heads x 64 p = 128, N = d_state, K = chunk.
//                CUDA cores scale x into a 128B-swizzled MN-major A tile; B comes straight from TMA (MN-major).
// chunk scan   : per (batch, chunk, group, 128-row block) one CTA computes CB = C.B^T ONCE into TMEM (it is shared by all
//                heads of the group) and then streams the heads of the group through a warp-specialised pipeline:
//                  compute warps : tcgen05.ld CB -> * exp(dAcs[l]-dAcs[s]) * dt[s], causal mask -> f16 -> swizzled smem (A operand)
//                  MMA warp      : Y  += S_kblock . X_kblock   (X tiles by TMA, MN-major B operand)
//                                  Z   = C . prev_state^T      (C tile reused from CB; prev state f16 by TMA)
//                  compute warps : y = Y + exp(dAcs[l]) * Z + D * x  -> f16
// The decay is always formed from the DIFFERENCE dAcs[l]-dAcs[s] <= 0 (never a ratio of exponentials).
// Every mbarrier wait is bounded; on a timeout the CTA records a code, drains and frees its tensor memory.
#include "ssd_common.cuh"
#include "tcgen05.cuh"

namespace b200 {

using namespace tc;

constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ float ex2_approx(float v)
{
	float r;
	asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v));
	return r;
}

// =====================================================================================================================
// chunk state
// =====================================================================================================================
namespace cstate {
constexpr int THREADS = 128;
constexpr int KB = 64;                      // l per K-block
constexpr int A_KB_BYTES = KB * 128 * 2;    // [2 atoms][64 l][64 m] f16 = 16 KiB
}  // namespace cstate

template <int NSTATE>
__global__ void __launch_bounds__(cstate::THREADS) ssd_chunk_state_tc_kernel(const __grid_constant__ CUtensorMap tmX,
	const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmS, const float* __restrict__ dt,
	const float* __restrict__ dacs, int64_t seqlen, int H, int G, int Q, int nchunks, uint32_t* err_word)
{
	using namespace cstate;
	constexpr int KA = NSTATE / 64;              // 64-wide n atoms
	constexpr int B_KB_BYTES = KA * KB * 128;    // per K-block: [KA atoms][64 l][64 n]
	extern __shared__ uint8_t smem_raw[];
	__shared__ uint64_t bar_in, bar_done;
	__shared__ uint32_t tmem_slot;
	__shared__ int abort_flag;
	__shared__ float s_scale[2][256];            // exp(dAcs[last] - dAcs[l]) * dt[l] for the two heads

	const int nkb = Q / KB;
	const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
	const uint32_t a_s = base;
	const uint32_t b_s = base + static_cast<uint32_t>(nkb) * A_KB_BYTES;
	uint8_t* a_gen = smem_raw + (base - smem_u32(smem_raw));

	const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
	const int hp = blockIdx.x % (H / 2);
	const int64_t bc = blockIdx.x / (H / 2);
	const int c = static_cast<int>(bc % nchunks);
	const int64_t b = bc / nchunks;
	const int h0 = hp * 2;
	const int g = h0 / (H / G);
	volatile int* abortp = &abort_flag;

	if (threadIdx.x == 0)
	{
		abort_flag = 0;
		mbar_init(smem_u32(&bar_in), 1);
		mbar_init(smem_u32(&bar_done), 1);
		fence_mbar_init();
	}
	if (warp == 0)
	{
		tmem_alloc(smem_u32(&tmem_slot), NSTATE);
		tmem_relinquish();
	}
	tc_fence_before();
	__syncthreads();
	tc_fence_after();
	const uint32_t tmem_base = tmem_slot;

	if (threadIdx.x == 0)
	{
		// raw x (both heads) and B tiles of the whole chunk; rows past the end of the sequence arrive as zeros
		prefetch_tmap(&tmX);
		prefetch_tmap(&tmB);
		const uint32_t in = smem_u32(&bar_in);
		mbar_arrive_expect_tx(in, static_cast<uint32_t>(nkb) * (A_KB_BYTES + B_KB_BYTES));
		for (int kb = 0; kb < nkb; ++kb)
		{
#pragma unroll
			for (int j = 0; j < 2; ++j)
				tma_load_3d(a_s + kb * A_KB_BYTES + j * (KB * 128), &tmX, in, (h0 + j) * 64, c * Q + kb * KB, static_cast<int>(b));
#pragma unroll
			for (int a = 0; a < KA; ++a)
				tma_load_3d(b_s + kb * B_KB_BYTES + a * (KB * 128), &tmB, in, g * NSTATE + a * 64, c * Q + kb * KB, static_cast<int>(b));
		}
	}
	// per-row scale factors while the tiles are in flight
	{
		const int64_t cb0 = ((b * H + h0) * nchunks + c) * static_cast<int64_t>(Q);
		for (int idx = threadIdx.x; idx < 2 * Q; idx += THREADS)
		{
			const int j = idx >= Q ? 1 : 0;
			const int l = idx - j * Q;
			const int64_t cbh = cb0 + static_cast<int64_t>(j) * nchunks * Q;
			s_scale[j][l] = __expf(dacs[cbh + Q - 1] - dacs[cbh + l]) * dt[cbh + l];
		}
	}
	__syncthreads();
	const bool loaded = mbar_wait(smem_u32(&bar_in), 0, abortp);
	if (loaded)
	{
		// scale x in place: the TMA layout (64 k-rows of 128 B per atom, 16-byte chunks XOR-swizzled by row) is the
		// MN-major A-operand layout already, and a row-wise scale keeps every element where it is
		const int chunk = threadIdx.x & 15;
		const int j = chunk >> 3, cj = chunk & 7;
		for (int l = threadIdx.x >> 4; l < Q; l += THREADS / 16)
		{
			const int kb = l >> 6, lk = l & 63;
			const uint32_t off = static_cast<uint32_t>(kb) * A_KB_BYTES + static_cast<uint32_t>(j) * (KB * 128) +
				static_cast<uint32_t>(lk) * 128 + (static_cast<uint32_t>(cj ^ (lk & 7)) << 4);
			Half8* p = reinterpret_cast<Half8*>(a_gen + off);
			float f[8];
			unpack8(*p, f);
			const float sc = s_scale[j][l];
#pragma unroll
			for (int e = 0; e < 8; ++e) f[e] *= sc;
			*p = pack8(f);
		}
	}
	fence_proxy_async_smem();
	__syncthreads();

	if (threadIdx.x == 0)
	{
		if (loaded)
		{
			tc_fence_after();
			constexpr uint32_t idesc = make_idesc_f16(128, NSTATE, 1, 1);
			for (int kb = 0; kb < nkb; ++kb)
			{
				const uint64_t a_desc = make_smem_desc_sw128(a_s + kb * A_KB_BYTES, KB * 128, 1024);
				const uint64_t b_desc = make_smem_desc_sw128(b_s + kb * B_KB_BYTES, KB * 128, 1024);
#pragma unroll
				for (int k = 0; k < KB / 16; ++k)
					mma_f16_ss(tmem_base, a_desc + static_cast<uint64_t>(k * 128), b_desc + static_cast<uint64_t>(k * 128), idesc,
						(kb | k) != 0 ? 1u : 0u);
			}
			mma_commit(smem_u32(&bar_done));
		}
		else
		{
			report_timeout(err_word, kErrScanWait);
		}
	}
	__syncwarp();
	if (loaded && mbar_wait(smem_u32(&bar_done), 0, abortp))
	{
		// the A tiles are dead now: each warp stages its 32 x NSTATE fp32 rows there and stores them with one TMA store
		tc_fence_after();
		uint8_t* stg = a_gen + warp * (32 * NSTATE * 4);
		const uint32_t t_row = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
#pragma unroll 1
		for (int cc = 0; cc < NSTATE / 32; ++cc)
		{
			uint32_t r[32];
			tmem_ld_32x32(t_row + static_cast<uint32_t>(cc * 32), r);
			tmem_ld_wait();
			float4* dst = reinterpret_cast<float4*>(stg + lane * (NSTATE * 4) + cc * 128);
#pragma unroll
			for (int v = 0; v < 8; ++v)
				dst[v] = make_float4(__uint_as_float(r[4 * v]), __uint_as_float(r[4 * v + 1]), __uint_as_float(r[4 * v + 2]),
					__uint_as_float(r[4 * v + 3]));
		}
		fence_proxy_async_smem();
		__syncwarp();
		if (lane == 0)
		{
			// states viewed as [b*nc*H*64 rows, NSTATE]; this warp owns 32 consecutive rows (head h0 + warp/2)
			const int row0 = static_cast<int>(((b * nchunks + c) * H + h0) * 64) + warp * 32;
			tma_store_2d(&tmS, a_s + warp * (32 * NSTATE * 4), 0, row0);
			bulk_commit_group();
			bulk_wait_group<0>();
		}
	}
	else if (lane == 0)
	{
		report_timeout(err_word, kErrScanWait);
	}
	if (*abortp)
		for (int i = 0; i < 2000; ++i) __nanosleep(1000);
	tc_fence_before();
	__syncthreads();
	if (warp == 0)
	{
		tc_fence_after();
		tmem_dealloc(tmem_base, NSTATE);
	}
}

// =====================================================================================================================
// chunk scan
// =====================================================================================================================
namespace cscan {
constexpr int LB = 128;   // output rows (l) per CTA
constexpr int KB = 64;    // s per K-block
constexpr int NCW = 16;        // compute warps: 4 TMEM lane quadrants x 2 K-block parities x 2 column halves
constexpr int MMA_B_WARP = 2 + NCW;      // second MMA-issuing warp (odd heads)
constexpr int THREADS = 96 + NCW * 32;  // warp 0 TMA, warp 1 MMA (CB, even heads), warps 2-17 compute, warp 18 MMA (odd heads)
constexpr int S_STAGE = LB * KB * 2;  // 16 KiB
constexpr int X_STAGE = KB * 64 * 2;  // 8 KiB
constexpr int H_FLOATS = 3 * 256;     // per-head dAcs | dt | colf rows of the chunk (Q <= 256)
constexpr uint32_t TMEM_COLS = 512;   // CB [0,256) | Y0 Z0 [256,384) | Y1 Z1 [384,512)

constexpr int Y_STAGE = 32 * 32;      // per-warp output staging: 32 rows x 16 f16 (32 B rows, dense)

// One ring of NST K-block stages, each holding the decayed-score tile S (written by the compute warps) and the X tile of the
// same K-block (TMA). One "full" barrier (8 compute-warp arrivals + the producer's expect_tx) and one "empty" barrier (one
// tcgen05.commit) per stage keep the MMA-issuing thread short: it is a single thread whose scalar instructions compete with
// the compute warps of its scheduler, and its wait/issue/commit sequence per K-block was the kernel's critical path.
// The S tiles of the ring start in the B region, which is dead once CB = C.B^T has been computed (the compute warps write
// their first S tile only after that) and run on into the S region: NST = NS + B_BYTES / S_STAGE stages, more than the
// K-blocks of one head, so the scores of head i+1 are produced while the tensor core still consumes those of head i.
template <int NSTATE, int NS, int NYB>
struct Layout
{
	static constexpr int KA = NSTATE / 64;
	static constexpr int C_BYTES = KA * LB * 128;      // [KA atoms][128 l][64 n]
	static constexpr int B_BYTES = KA * 256 * 128;     // [KA atoms][256 s][64 n]
	static constexpr int P_BYTES = KA * 64 * 128;      // [KA atoms][64 p][64 n]
	static constexpr int OFF_C = 0;
	static constexpr int OFF_B = OFF_C + C_BYTES;
	static constexpr int OFF_S = OFF_B + B_BYTES;
	static constexpr int NST = NS + B_BYTES / S_STAGE;
	static constexpr int OFF_X = OFF_S + NS * S_STAGE;
	static constexpr int OFF_P = OFF_X + NST * X_STAGE;
	static constexpr int OFF_H = OFF_P + 2 * P_BYTES;
	static constexpr int OFF_Y = OFF_H + 2 * H_FLOATS * 4;   // [NCW compute warps][NYB buffers][Y_STAGE]
	static constexpr int TOTAL = OFF_Y + NCW * NYB * Y_STAGE + 1024;
	static_assert(TOTAL <= 232448, "shared memory layout exceeds the per-CTA limit");
	// byte offsets of stage `st`: S tiles are contiguous from the start of the B region
	static __host__ __device__ constexpr int s_off(int st) { return OFF_B + st * S_STAGE; }
	static __host__ __device__ constexpr int x_off(int st) { return OFF_X + st * X_STAGE; }
};
}  // namespace cscan

template <int NSTATE, int NS, int NYB>
__global__ void __launch_bounds__(cscan::THREADS, 1) ssd_chunk_scan_tc_kernel(const __grid_constant__ CUtensorMap tmX,
	const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmP,
	const __grid_constant__ CUtensorMap tmY, const float* __restrict__ D,
	const float* __restrict__ dt, const float* __restrict__ dacs, const float* __restrict__ colf, int64_t seqlen, int H, int G,
	int Q, int nchunks, int heads_per_cta, uint32_t* err_word)
{
	using namespace cscan;
	using L = Layout<NSTATE, NS, NYB>;
	constexpr int KA = L::KA;
	constexpr int NST = L::NST;
	extern __shared__ uint8_t smem_raw[];
	__shared__ uint64_t bar_in, bar_cb, k_full[NST], k_empty[NST], p_full[2], p_empty[2], acc_full[2],
		acc_empty[2], h_full[2], h_empty[2];
	__shared__ uint32_t tmem_slot;
	__shared__ int abort_flag;

	const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
	uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
	const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
	volatile int* abortp = &abort_flag;

	// work decode: blockIdx.x -> (batch, chunk, group, l-block); blockIdx.y -> slice of the group's heads
	const int lblocks = Q / LB;
	const int lb = lblocks - 1 - static_cast<int>(blockIdx.x % lblocks);  // heavier blocks first
	int64_t rest = blockIdx.x / lblocks;
	const int g = static_cast<int>(rest % G);
	rest /= G;
	const int c = static_cast<int>(rest % nchunks);
	const int64_t b = rest / nchunks;
	const int hpg = H / G;
	const int h_begin = g * hpg + static_cast<int>(blockIdx.y) * heads_per_cta;
	const int h_end = min(h_begin + heads_per_cta, (g + 1) * hpg);
	const int nheads = h_end - h_begin;
	const int l0 = lb * LB;
	const int s_count = l0 + LB;        // causal extent of this row block
	const int nkb = s_count / KB;       // 2 or 4
	const int valid = static_cast<int>(min(static_cast<int64_t>(Q), seqlen - static_cast<int64_t>(c) * Q));

	if (threadIdx.x == 0)
	{
		abort_flag = 0;
		mbar_init(smem_u32(&bar_in), 1);
		mbar_init(smem_u32(&bar_cb), 1);
		for (int i = 0; i < NST; ++i) { mbar_init(smem_u32(&k_full[i]), 9); mbar_init(smem_u32(&k_empty[i]), 1); }
		for (int i = 0; i < 2; ++i)
		{
			mbar_init(smem_u32(&p_full[i]), 1);
			mbar_init(smem_u32(&p_empty[i]), 1);
			mbar_init(smem_u32(&acc_full[i]), 1);
			mbar_init(smem_u32(&acc_empty[i]), NCW);
			mbar_init(smem_u32(&h_full[i]), 1);
			mbar_init(smem_u32(&h_empty[i]), NCW);
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

	if (nheads <= 0 || l0 >= valid) goto role_done;  // nothing to produce (uniform across the CTA)

	if (warp == 0)
	{
		if (lane == 0)
		{
			prefetch_tmap(&tmX); prefetch_tmap(&tmB); prefetch_tmap(&tmC); prefetch_tmap(&tmP);
			const uint32_t in = smem_u32(&bar_in);
			mbar_arrive_expect_tx(in, static_cast<uint32_t>(KA * (LB + s_count) * 128));
#pragma unroll
			for (int a = 0; a < KA; ++a)
			{
				for (int j = 0; j < LB / 64; ++j)
					tma_load_3d(base + L::OFF_C + a * (LB * 128) + j * 8192, &tmC, in, g * NSTATE + a * 64, c * Q + l0 + j * 64,
						static_cast<int>(b));
				for (int j = 0; j < s_count / 64; ++j)
					tma_load_3d(base + L::OFF_B + a * (256 * 128) + j * 8192, &tmB, in, g * NSTATE + a * 64, c * Q + j * 64,
						static_cast<int>(b));
			}
			int kst = 0;
			uint32_t kphase = 0;
			for (int i = 0; i < nheads; ++i)
			{
				const int h = h_begin + i;
				const int buf = i & 1;
				// per-head rows of dAcs, dt and colf for this chunk
				if (!mbar_wait(smem_u32(&h_empty[buf]), ((i >> 1) & 1) ^ 1u, abortp))
				{
					report_timeout(err_word, kErrProducerWait);
					goto role_done;
				}
				{
					const int64_t cbase = ((b * H + h) * nchunks + c) * static_cast<int64_t>(Q);
					const uint32_t hb = base + L::OFF_H + buf * (H_FLOATS * 4);
					const uint32_t bytes = static_cast<uint32_t>(Q) * 4;
					mbar_arrive_expect_tx(smem_u32(&h_full[buf]), 3 * bytes);
					bulk_load_1d(hb, dacs + cbase, bytes, smem_u32(&h_full[buf]));
					bulk_load_1d(hb + 1024, dt + cbase, bytes, smem_u32(&h_full[buf]));
					bulk_load_1d(hb + 2048, colf + cbase, bytes, smem_u32(&h_full[buf]));
				}
				for (int kb = 0; kb < nkb; ++kb)
				{
					if (!mbar_wait(smem_u32(&k_empty[kst]), kphase ^ 1u, abortp))
					{
						report_timeout(err_word, kErrProducerWait);
						goto role_done;
					}
					mbar_arrive_expect_tx(smem_u32(&k_full[kst]), X_STAGE);
					tma_load_3d(base + L::x_off(kst), &tmX, smem_u32(&k_full[kst]), h * 64, c * Q + kb * KB, static_cast<int>(b));
					if (++kst == NST) { kst = 0; kphase ^= 1u; }
				}
				if (!mbar_wait(smem_u32(&p_empty[buf]), ((i >> 1) & 1) ^ 1u, abortp))
				{
					report_timeout(err_word, kErrProducerWait);
					goto role_done;
				}
				mbar_arrive_expect_tx(smem_u32(&p_full[buf]), L::P_BYTES);
				const int prow = static_cast<int>(((b * nchunks + c) * H + h) * 64);
#pragma unroll
				for (int a = 0; a < KA; ++a)
					tma_load_2d(base + L::OFF_P + buf * L::P_BYTES + a * 8192, &tmP, smem_u32(&p_full[buf]), a * 64, prow);
			}
		}
	}
	else if (warp == 1)
	{
		if (lane == 0)
		{
			if (!mbar_wait(smem_u32(&bar_in), 0, abortp))
			{
				report_timeout(err_word, kErrMmaWaitFull);
				goto role_done;
			}
			tc_fence_after();
			{
				// CB[l, s] = sum_n C[l,n] B[s,n]  (N = s_count columns)
				const uint32_t idesc_cb = make_idesc_f16(LB, s_count, 0);
#pragma unroll
				for (int a = 0; a < KA; ++a)
				{
					const uint64_t a_desc = make_smem_desc_sw128(base + L::OFF_C + a * (LB * 128), 16, 1024);
					const uint64_t b_desc = make_smem_desc_sw128(base + L::OFF_B + a * (256 * 128), 16, 1024);
#pragma unroll
					for (int k = 0; k < 4; ++k)
						mma_f16_ss(tmem_base, a_desc + static_cast<uint64_t>(k * 2), b_desc + static_cast<uint64_t>(k * 2), idesc_cb,
							(a | k) != 0 ? 1u : 0u);
				}
				mma_commit(smem_u32(&bar_cb));
			}
		}
		// falls through to the head loop below as the issuer of the even heads
	}
	if ((warp == 1 || warp == MMA_B_WARP) && lane == 0 && !*abortp)
	{
		// Two MMA-issuing threads, even heads (accumulator 0) and odd heads (accumulator 1): a head's wait / descriptor /
		// tcgen05.mma / commit sequence is a few hundred dependent scalar instructions of ONE thread that shares its scheduler
		// with compute warps, about as long as the compute warps need for a head's scores. The two threads' MMAs touch
		// different accumulators and different ring stages, so they need no ordering between each other.
		const int par = warp == 1 ? 0 : 1;
		constexpr uint32_t idesc_y = make_idesc_f16(LB, 64, 1);  // B operand (x) is MN-major
		constexpr uint32_t idesc_z = make_idesc_f16(LB, 64, 0);
		const uint64_t s_desc0 = make_smem_desc_sw128(base + L::s_off(0), 16, 1024);
		const uint64_t x_desc0 = make_smem_desc_sw128(base + L::x_off(0), KB * 128, 1024);
		const uint32_t y_tmem = tmem_base + 256u + static_cast<uint32_t>(par * 128);
		const uint32_t z_tmem = y_tmem + 64u;
		bool ok = par == 0 || mbar_wait(smem_u32(&bar_in), 0, abortp);  // C tile resident (the even issuer waited already)
		if (!ok) report_timeout(err_word, kErrMmaWaitFull);
		tc_fence_after();
		// ring position of K-block 0 of head `par`
		int kst = (par * nkb) % NST;
		uint32_t kphase = static_cast<uint32_t>((par * nkb) / NST) & 1u;
		for (int i = par; ok && i < nheads; i += 2)
		{
			const uint32_t use = static_cast<uint32_t>(i >> 1) & 1u;  // parity of this accumulator's use count
			if (!mbar_wait(smem_u32(&acc_empty[par]), use ^ 1u, abortp))
			{
				report_timeout(err_word, kErrMmaWaitTmem);
				break;
			}
			tc_fence_after();
			for (int kb = 0; kb < nkb; ++kb)
			{
				if (!mbar_wait(smem_u32(&k_full[kst]), kphase, abortp))
				{
					report_timeout(err_word, kErrMmaWaitFull);
					ok = false;
					break;
				}
				tc_fence_after();
				// descriptors address shared memory in 16-byte units: stage st is st * (stage bytes / 16) further on
				const uint64_t a_desc = s_desc0 + static_cast<uint64_t>(kst * (S_STAGE >> 4));
				const uint64_t b_desc = x_desc0 + static_cast<uint64_t>(kst * (X_STAGE >> 4));
#pragma unroll
				for (int k = 0; k < KB / 16; ++k)
					mma_f16_ss(y_tmem, a_desc + static_cast<uint64_t>(k * 2), b_desc + static_cast<uint64_t>(k * 128), idesc_y,
						(kb | k) != 0 ? 1u : 0u);
				mma_commit(smem_u32(&k_empty[kst]));
				if (++kst == NST) { kst = 0; kphase ^= 1u; }
			}
			if (!ok) break;
			if (!mbar_wait(smem_u32(&p_full[par]), use, abortp))
			{
				report_timeout(err_word, kErrMmaWaitFull);
				break;
			}
			tc_fence_after();
#pragma unroll
			for (int a = 0; a < KA; ++a)
			{
				const uint64_t a_desc = make_smem_desc_sw128(base + L::OFF_C + a * (LB * 128), 16, 1024);
				const uint64_t b_desc = make_smem_desc_sw128(base + L::OFF_P + par * L::P_BYTES + a * 8192, 16, 1024);
#pragma unroll
				for (int k = 0; k < 4; ++k)
					mma_f16_ss(z_tmem, a_desc + static_cast<uint64_t>(k * 2), b_desc + static_cast<uint64_t>(k * 2), idesc_z,
						(a | k) != 0 ? 1u : 0u);
			}
			mma_commit(smem_u32(&p_empty[par]));
			mma_commit(smem_u32(&acc_full[par]));
			// skip the other issuer's head
			kst += nkb;
			if (kst >= NST) { kst -= NST; kphase ^= 1u; }
		}
	}
	else if (warp >= 2 && warp < 2 + NCW)
	{
		const int q = warp & 3;           // TMEM lane quadrant
		const int cw = warp - 2;          // compute warp index 0..15
		const int kpar = (cw >> 2) & 1;   // parity of the K-blocks this warp scales
		const int chalf = cw >> 3;        // which 32-column half of a K-block
		const int r = q * 32 + lane;      // row inside the block
		const int l = l0 + r;
		const int wrow0 = l0 + q * 32;    // first row of this warp
		const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
		uint8_t* ystg = gen + L::OFF_Y + cw * (NYB * Y_STAGE);
		const uint32_t ystg_s = base + L::OFF_Y + cw * (NYB * Y_STAGE);
		float dl2_prev = 0.f;
		uint32_t nstore = 0;
		bool cb_ready = false;
		if (lane == 0) prefetch_tmap(&tmY);

		// y[l, h, cw*4 .. +15 columns] = Y + exp(dAcs[l]) * Z, staged per warp and written by one TMA store (rows past the
		// end of the sequence are clipped by the store). The D*x skip term is already inside Y: D sits on the diagonal of S.
		auto epilogue = [&](int i, float dl2) -> bool {
			const int buf = i & 1;
			const int h = h_begin + i;
			const int ecol = (cw >> 2) * 16;  // this warp's 16 of the 64 head columns
			if (!mbar_wait(smem_u32(&acc_full[buf]), (i >> 1) & 1, abortp)) return false;
			tc_fence_after();
			uint32_t yr[16], zr[16];
			const uint32_t col = 256u + static_cast<uint32_t>(buf * 128 + ecol);
			tmem_ld_32x16(t_lane + col, yr);
			tmem_ld_32x16(t_lane + col + 64u, zr);
			if (lane == 0) bulk_wait_group_read<NYB - 1>();  // the staging buffer about to be rewritten has been read
			tmem_ld_wait();
			tc_fence_before();
			__syncwarp();
			if (lane == 0) mbar_arrive(smem_u32(&acc_empty[buf]));
			const float dec = ex2_approx(dl2);
			const uint32_t sb = (nstore % NYB) * Y_STAGE;
#pragma unroll
			for (int v = 0; v < 2; ++v)
			{
				float o[8];
#pragma unroll
				for (int e = 0; e < 8; ++e) o[e] = fmaf(dec, __uint_as_float(zr[v * 8 + e]), __uint_as_float(yr[v * 8 + e]));
				*reinterpret_cast<Half8*>(ystg + sb + lane * 32 + v * 16) = pack8(o);
			}
			fence_proxy_async_smem();
			__syncwarp();
			if (lane == 0)
			{
				tma_store_3d(&tmY, ystg_s + sb, h * 64 + ecol, c * Q + wrow0, static_cast<int>(b));
				bulk_commit_group();
			}
			++nstore;
			return true;
		};

		for (int i = 0; i < nheads; ++i)
		{
			const int h = h_begin + i;
			const int buf = i & 1;
			const float* hd = reinterpret_cast<const float*>(gen + L::OFF_H + buf * (H_FLOATS * 4));  // dAcs | dt | colf
			const float dh = D ? __ldg(D + h) : 0.f;
			if (!mbar_wait(smem_u32(&h_full[buf]), (i >> 1) & 1, abortp))
			{
				if (lane == 0) report_timeout(err_word, kErrScanWait);
				goto role_done;
			}
			const float dl2 = hd[l] * kLog2e;
			for (int kb = kpar; kb < nkb; kb += 2)
			{
				// stage and phase of K-block (i, kb) in the ring: this warp visits every second K-block
				const int kbc = i * nkb + kb;
				const int ss = kbc % NST;
				if (!mbar_wait(smem_u32(&k_empty[ss]), ((kbc / NST) & 1) ^ 1u, abortp))
				{
					if (lane == 0) report_timeout(err_word, kErrScanWait);
					goto role_done;
				}
				if (!cb_ready)
				{
					if (!mbar_wait(smem_u32(&bar_cb), 0, abortp))
					{
						if (lane == 0) report_timeout(err_word, kErrScanWait);
						goto role_done;
					}
					cb_ready = true;
				}
				tc_fence_after();
				uint8_t* srow = gen + L::s_off(ss) + r * 128;
				const int s_first = kb * KB;          // first column of the 64-wide K-block
				const int s0 = s_first + chalf * 32;  // first of this warp's 32 columns
				if (s0 > wrow0 + 31)
				{
					// these 32 x 32 scores lie above the diagonal
					Half8 zero;
#pragma unroll
					for (int e = 0; e < 4; ++e) zero.h[e] = __floats2half2_rn(0.f, 0.f);
#pragma unroll
					for (int v = 0; v < 4; ++v) *reinterpret_cast<Half8*>(srow + (((chalf * 4 + v) ^ (r & 7)) << 4)) = zero;
				}
				else
				{
					uint32_t cbv[32];
					tmem_ld_32x32(t_lane + static_cast<uint32_t>(s0), cbv);
					if (s_first + KB - 1 <= wrow0 - 1)
					{
						// K-block entirely below the diagonal: decay = exp(dAcs[l] - dAcs[block end]) * colf[s], both factors <= 1
						const float rk = ex2_approx(fmaf(hd[s_first + KB - 1], -kLog2e, dl2));
						const float4* cfp = reinterpret_cast<const float4*>(hd + 512 + s0);
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
							*reinterpret_cast<Half8*>(srow + (((chalf * 4 + v) ^ (r & 7)) << 4)) = pack8(o);
						}
					}
					else
					{
						// crossed by the diagonal: exact exp of the (non-positive) difference, causal mask, and the D skip
						// connection as S[l,l] += D (so that S.x carries D*x)
						const float4* dsp = reinterpret_cast<const float4*>(hd + s0);
						const float4* dtp = reinterpret_cast<const float4*>(hd + 256 + s0);
						tmem_ld_wait();
#pragma unroll
						for (int v = 0; v < 4; ++v)  // 8 s-values -> one 16-byte chunk
						{
							float o[8];
#pragma unroll
							for (int hq = 0; hq < 2; ++hq)
							{
								const float4 ds = dsp[v * 2 + hq];
								const float4 dv = dtp[v * 2 + hq];
								const float dsa[4] = { ds.x, ds.y, ds.z, ds.w };
								const float dta[4] = { dv.x, dv.y, dv.z, dv.w };
#pragma unroll
								for (int e = 0; e < 4; ++e)
								{
									const int j = v * 8 + hq * 4 + e;
									const float w = ex2_approx(fmaf(dsa[e], -kLog2e, dl2)) * dta[e];
									float val = (s0 + j <= l) ? __uint_as_float(cbv[j]) * w : 0.f;
									if (s0 + j == l) val += dh;
									o[hq * 4 + e] = val;
								}
							}
							*reinterpret_cast<Half8*>(srow + (((chalf * 4 + v) ^ (r & 7)) << 4)) = pack8(o);
						}
					}
				}
				fence_proxy_async_smem();
				__syncwarp();
				if (lane == 0) mbar_arrive(smem_u32(&k_full[ss]));
			}
			// this warp no longer reads the per-head rows
			__syncwarp();
			if (lane == 0) mbar_arrive(smem_u32(&h_empty[buf]));
			if (i > 0 && !epilogue(i - 1, dl2_prev))
			{
				if (lane == 0) report_timeout(err_word, kErrEpilogueWait);
				goto role_done;
			}
			dl2_prev = dl2;
		}
		if (!epilogue(nheads - 1, dl2_prev))
		{
			if (lane == 0) report_timeout(err_word, kErrEpilogueWait);
		}
		if (lane == 0) bulk_wait_group<0>();  // stores must have left shared memory before the CTA exits
	}

role_done:
	__syncwarp();
	if (*abortp)
		for (int i = 0; i < 2000; ++i) __nanosleep(1000);
	tc_fence_before();
	__syncthreads();
	if (warp == 1)
	{
		tc_fence_after();
		tmem_dealloc(tmem_base, TMEM_COLS);
	}
}

// =====================================================================================================================
// host side
// =====================================================================================================================

bool ssd_tc_supported(const SsdDims& d, const void* x, int64_t xs, const void* Bm, int64_t bs, const void* Cm, int64_t cs, const void* y,
	int64_t ys)
{
	if (d.P != 64 || (d.N != 64 && d.N != 128) || (d.Q != 128 && d.Q != 256)) return false;
	if ((d.H / d.G) % 2 != 0) return false;  // head pairs must share a group
	if (xs % 8 || bs % 8 || cs % 8 || ys % 8) return false;
	if (!aligned16(x) || !aligned16(Bm) || !aligned16(Cm) || !aligned16(y)) return false;
	if (d.batch > 0x7fffffffLL || d.seqlen > 0x7fffffffLL) return false;
	if (d.batch * d.nchunks * d.H * 64 > 0x7fffffffLL) return false;  // prev-state row index is a 32-bit TMA coordinate
	return true;
}

int ssd_chunk_state_tc(const __half* x, int64_t xs, const __half* Bm, int64_t bs, const SsdDims& d, const SsdWorkspace& w, cudaStream_t st)
{
	CUtensorMap tmX, tmB, tmS;
	const uint64_t L = static_cast<uint64_t>(d.seqlen), Bt = static_cast<uint64_t>(d.batch);
	int rc = tmap_3d_f16(&tmX, x, static_cast<uint64_t>(d.H) * 64, L, Bt, static_cast<uint64_t>(xs), L * xs, 64, 64);
	if (rc) return rc;
	rc = tmap_3d_f16(&tmB, Bm, static_cast<uint64_t>(d.G) * d.N, L, Bt, static_cast<uint64_t>(bs), L * bs, 64, 64);
	if (rc) return rc;
	rc = tmap_2d_f32_linear(&tmS, w.states, static_cast<uint64_t>(d.batch) * d.nchunks * d.H * 64, static_cast<uint64_t>(d.N),
		static_cast<uint64_t>(d.N), static_cast<uint32_t>(d.N), 32);
	if (rc) return rc;
	const int nkb = d.Q / 64;
	const unsigned grid = static_cast<unsigned>(d.batch * d.nchunks * (d.H / 2));
	if (d.N == 64)
	{
		const int smem = nkb * (cstate::A_KB_BYTES + 64 * 128) + 1024;
		static bool smem_ok[64] = {};
		B200_CUDA_TRY(allow_dynamic_smem(ssd_chunk_state_tc_kernel<64>, 4 * (cstate::A_KB_BYTES + 64 * 128) + 1024, smem_ok));
		ssd_chunk_state_tc_kernel<64><<<grid, cstate::THREADS, smem, st>>>(tmX, tmB, tmS, w.dt, w.dacs, d.seqlen, d.H, d.G, d.Q, d.nchunks,
			device_error_word());
	}
	else
	{
		const int smem = nkb * (cstate::A_KB_BYTES + 2 * 64 * 128) + 1024;
		static bool smem_ok[64] = {};
		B200_CUDA_TRY(allow_dynamic_smem(ssd_chunk_state_tc_kernel<128>, 4 * (cstate::A_KB_BYTES + 2 * 64 * 128) + 1024, smem_ok));
		ssd_chunk_state_tc_kernel<128><<<grid, cstate::THREADS, smem, st>>>(tmX, tmB, tmS, w.dt, w.dacs, d.seqlen, d.H, d.G, d.Q, d.nchunks,
			device_error_word());
	}
	B200_LAUNCH_CHECK();
	return B200_OK;
}

int ssd_chunk_scan_tc(const __half* x, int64_t xs, const __half* Bm, int64_t bs, const __half* Cm, int64_t cs, const float* D, __half* y,
	int64_t ys, const SsdDims& d, const SsdWorkspace& w, cudaStream_t st)
{
	CUtensorMap tmX, tmB, tmC, tmP, tmY;
	const uint64_t L = static_cast<uint64_t>(d.seqlen), Bt = static_cast<uint64_t>(d.batch);
	int rc = tmap_3d_f16(&tmX, x, static_cast<uint64_t>(d.H) * 64, L, Bt, static_cast<uint64_t>(xs), L * xs, 64, 64);
	if (rc) return rc;
	rc = tmap_3d_f16(&tmB, Bm, static_cast<uint64_t>(d.G) * d.N, L, Bt, static_cast<uint64_t>(bs), L * bs, 64, 64);
	if (rc) return rc;
	rc = tmap_3d_f16(&tmC, Cm, static_cast<uint64_t>(d.G) * d.N, L, Bt, static_cast<uint64_t>(cs), L * cs, 64, 64);
	if (rc) return rc;
	rc = tmap_2d_f16(&tmP, w.prev16, static_cast<uint64_t>(d.batch) * d.nchunks * d.H * 64, static_cast<uint64_t>(d.N),
		static_cast<uint64_t>(d.N), 64, 64);
	if (rc) return rc;
	rc = tmap_3d_f16_linear(&tmY, y, static_cast<uint64_t>(d.H) * 64, L, Bt, static_cast<uint64_t>(ys), L * ys, 16, 32);
	if (rc) return rc;
	const int lblocks = d.Q / cscan::LB;
	const int hpg = d.H / d.G;
	// enough CTAs to fill the machine, but as many heads per CTA as possible so that CB is computed rarely
	const int64_t base_ctas = d.batch * d.nchunks * d.G * lblocks;
	int hpc = hpg;
	while (hpc > 4 && base_ctas * cdiv(hpg, hpc) < 2 * kNumSMs) hpc = (hpc + 1) / 2;
	const dim3 grid(static_cast<unsigned>(base_ctas), static_cast<unsigned>(cdiv(hpg, hpc)));
	if (d.N == 64)
	{
		using Lt = cscan::Layout<64, 4, 1>;
		static bool smem_ok[64] = {};
		B200_CUDA_TRY(allow_dynamic_smem(ssd_chunk_scan_tc_kernel<64, 4, 1>, Lt::TOTAL, smem_ok));
		ssd_chunk_scan_tc_kernel<64, 4, 1><<<grid, cscan::THREADS, Lt::TOTAL, st>>>(tmX, tmB, tmC, tmP, tmY, D, w.dt, w.dacs, w.colf, d.seqlen,
			d.H, d.G, d.Q, d.nchunks, hpc, device_error_word());
	}
	else
	{
		using Lt = cscan::Layout<128, 1, 1>;
		static bool smem_ok[64] = {};
		B200_CUDA_TRY(allow_dynamic_smem(ssd_chunk_scan_tc_kernel<128, 1, 1>, Lt::TOTAL, smem_ok));
		ssd_chunk_scan_tc_kernel<128, 1, 1><<<grid, cscan::THREADS, Lt::TOTAL, st>>>(tmX, tmB, tmC, tmP, tmY, D, w.dt, w.dacs, w.colf, d.seqlen,
			d.H, d.G, d.Q, d.nchunks, hpc, device_error_word());
	}
	B200_LAUNCH_CHECK();
	return B200_OK;
}

}  // namespace b200
