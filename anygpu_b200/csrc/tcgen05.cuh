// Thin inline-PTX layer for the Blackwell (sm_100a) data path used by the tensor-core kernels:
// mbarrier (with BOUNDED waits), TMA tiled loads, tensor-memory allocation, tcgen05.mma / commit / ld,
// and the shared-memory / instruction descriptor encodings.
#pragma once
#include <cuda.h>  // CUtensorMap (types only; the encode function is fetched from the driver at run time)
#include "common.cuh"

namespace b200 {
namespace tc {

// A wait gives up after this many polls, sets the abort flag and lets the kernel unwind (free TMEM, return).
constexpr uint32_t kSpinLimit = 1u << 22;

// Codes written to the device error word (upper 16 bits: site, lower 16 bits: blockIdx.x).
enum : uint32_t
{
	kErrProducerWait = 1,
	kErrMmaWaitFull = 2,
	kErrMmaWaitTmem = 3,
	kErrEpilogueWait = 4,
	kErrScanWait = 5
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
	asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes)
{
	asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
	asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
	uint32_t ok;
	asm volatile(
		"{\n\t.reg .pred p;\n\t"
		"mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
		"selp.b32 %0, 1, 0, p;\n\t}"
		: "=r"(ok)
		: "r"(bar), "r"(parity)
		: "memory");
	return ok != 0;
}

// Bounded wait. Returns false when it gave up (or another role already aborted); never spins forever.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, uint32_t limit = kSpinLimit)
{
	for (uint32_t i = 0; i < limit; ++i)
	{
		if (mbar_try_wait(bar, parity)) return true;
		if ((i & 255u) == 255u && *abort_flag) return false;
	}
	*abort_flag = 1;
	return false;
}

__device__ __forceinline__ void report_timeout(uint32_t* err_word, uint32_t site)
{
	if (err_word) atomicCAS(err_word, 0u, (site << 16) | (blockIdx.x & 0xffffu));
}

// ---- TMA ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* m)
{
	asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// 2-D tiled load global -> shared, completion counted in bytes on `bar`. x = innermost coordinate (elements).
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* m, uint32_t bar, int x, int y)
{
	asm volatile(
		"cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
		::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y)
		: "memory");
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* m, uint32_t bar, int x, int y, int z)
{
	asm volatile(
		"cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
		::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y), "r"(z)
		: "memory");
}

// Asks for the tile to be brought into L2 (no destination in shared memory, nothing to wait for).
__device__ __forceinline__ void tma_prefetch_3d(const CUtensorMap* m, int x, int y, int z)
{
	asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global.tile [%0, {%1, %2, %3}];"
		::"l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y), "r"(z)
		: "memory");
}

// Tiled stores shared -> global (bulk async-group completion). Rows / columns outside the tensor are clipped.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, uint32_t src, int x, int y)
{
	asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
		::"l"(reinterpret_cast<uint64_t>(m)), "r"(src), "r"(x), "r"(y)
		: "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* m, uint32_t src, int x, int y, int z)
{
	asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
		::"l"(reinterpret_cast<uint64_t>(m)), "r"(src), "r"(x), "r"(y), "r"(z)
		: "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Waits until at most N of this thread's bulk groups still READ their shared-memory source.
template <int N>
__device__ __forceinline__ void bulk_wait_group_read()
{
	asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
// Waits until at most N of this thread's bulk groups are still in flight at all (global writes performed).
template <int N>
__device__ __forceinline__ void bulk_wait_group()
{
	asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// 1-D bulk copy global -> shared (both addresses 16-byte aligned, size a multiple of 16 bytes), completion on `bar`.
__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar)
{
	asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
		::"r"(dst), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar)
		: "memory");
}

// ---- tensor memory -----------------------------------------------------------------------------------------
// Whole-warp calls. ncols: power of two in [32, 512].
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols)
{
	asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish()
{
	asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols)
{
	asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem] . B[smem], f16 inputs, fp32 accumulate. One thread issues.
__device__ __forceinline__ void mma_f16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
	asm volatile(
		"{\n\t.reg .pred p;\n\t"
		"setp.ne.b32 p, %4, 0;\n\t"
		"tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
		::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
		: "memory");
}
// Arrives on `bar` when every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void mma_commit(uint32_t bar)
{
	asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// 32 lanes x 32 consecutive fp32 columns -> 32 registers per thread (thread i of the warp = lane base + i).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t* r)
{
	asm volatile(
		"tcgen05.ld.sync.aligned.32x32b.x32.b32 "
		"{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
		"%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
		: "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
		  "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
		  "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
		  "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
		: "r"(taddr)
		: "memory");
}
// 32 lanes x 16 consecutive fp32 columns.
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t* r)
{
	asm volatile(
		"tcgen05.ld.sync.aligned.32x32b.x16.b32 "
		"{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
		: "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
		  "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
		: "r"(taddr)
		: "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---- CTA pairs (cta_group::2): cluster rank, peer addresses, pair-wide MMA ---------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank()
{
	uint32_t r;
	asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
	return r;
}
// shared::cluster address of `local_addr` (a shared::cta address of this CTA) inside CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank)
{
	uint32_t r;
	asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
	return r;
}
__device__ __forceinline__ void cluster_sync()
{
	asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// arrive on an mbarrier that may live in the peer CTA (shared::cluster address)
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr)
{
	asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// 2-D tiled load into THIS CTA's shared memory whose completion bytes are counted on an mbarrier of the pair's leader CTA
// (no multicast: each CTA of the pair fetches its own tile)
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* m, uint32_t leader_bar, int x, int y)
{
	asm volatile(
		"cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
		::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(leader_bar), "r"(x), "r"(y)
		: "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_dst, uint32_t ncols)
{
	asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair()
{
	asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols)
{
	asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// D[tmem of both CTAs] (+)= A . B with M = 256 split over the pair; issued by one thread of the leader CTA
__device__ __forceinline__ void mma_f16_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
	asm volatile(
		"{\n\t.reg .pred p;\n\t"
		"setp.ne.b32 p, %4, 0;\n\t"
		"tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
		::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
		: "memory");
}
// arrives on the mbarrier at the same shared-memory offset in every CTA of `cta_mask` once the pair's MMAs issued so far completed
__device__ __forceinline__ void mma_commit_pair(uint32_t bar, uint16_t cta_mask)
{
	asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
		::"r"(bar), "h"(cta_mask)
		: "memory");
}

// ---- descriptors -------------------------------------------------------------------------------------------
// Instruction descriptor, kind::f16: D fp32, A/B f16, A K-major; B K-major (b_mn = 0) or MN-major (b_mn = 1).
__host__ __device__ constexpr uint32_t make_idesc_f16(int M, int N, int b_mn, int a_mn = 0)
{
	return (1u << 4)                                   // D format fp32
		| (0u << 7) | (0u << 10)                       // A, B format f16
		| (static_cast<uint32_t>(a_mn) << 15)          // A major
		| (static_cast<uint32_t>(b_mn) << 16)          // B major
		| (static_cast<uint32_t>(N >> 3) << 17)        // N / 8
		| (static_cast<uint32_t>(M >> 4) << 24);       // M / 16
}

// Shared-memory matrix descriptor for a 128-byte-swizzled operand tile (tile base 1024-byte aligned).
//   K-major : rows of 64 f16 (128 B); 8-row groups 1024 B apart  -> sbo = 1024, lbo unused (1).
//   MN-major: k-rows of 64 f16 along MN (128 B); 8-k-row groups sbo bytes apart, 64-wide MN blocks lbo bytes apart.
__device__ __forceinline__ uint64_t make_smem_desc_sw128(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes)
{
	uint64_t d = 0;
	d |= static_cast<uint64_t>((saddr & 0x3ffffu) >> 4);
	d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3fffu) << 16;
	d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3fffu) << 32;
	d |= 1ull << 46;  // descriptor version for sm_100
	d |= 2ull << 61;  // SWIZZLE_128B
	return d;
}

}  // namespace tc

// ---- host: 128-byte-swizzled f16 tensor maps (encoded through the driver entry point, cached by key) -------------
// 2-D tensor [rows, cols], row stride ld (elements); box = box_cols x box_rows.
int tmap_2d_f16(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld_elems, uint32_t box_cols,
	uint32_t box_rows);
// 3-D tensor [d2, d1, d0] (d0 innermost), element strides s1 (between d1 rows) and s2 (between d2 slabs); box d0 x d1 x 1.
// Out-of-range coordinates in any dimension read zeros, so a per-sequence row tail never picks up the next sequence.
int tmap_3d_f16(CUtensorMap* out, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t s1_elems, uint64_t s2_elems,
	uint32_t box0, uint32_t box1);

// 128-byte-swizzled fp32 map of a 3-D tensor (box of box0 <= 32 floats x box1 rows x 1).
int tmap_3d_f32(CUtensorMap* out, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t s1_elems, uint64_t s2_elems,
	uint32_t box0, uint32_t box1);

// Unswizzled maps used by TMA STORES of small per-warp tiles (rows of box0 elements, dense in shared memory).
int tmap_3d_f16_linear(CUtensorMap* out, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t s1_elems,
	uint64_t s2_elems, uint32_t box0, uint32_t box1);
int tmap_2d_f32_linear(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld_elems, uint32_t box_cols,
	uint32_t box_rows);

}  // namespace b200
