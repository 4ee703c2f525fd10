// Host-side TMA tensor-map construction. The encode function comes from the driver through
// cudaGetDriverEntryPoint, so the library links against the CUDA runtime only.
#include <cstring>
#include <mutex>
#include <unordered_map>

#include "tcgen05.cuh"

namespace b200 {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
	const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
	CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn()
{
	static EncodeTiledFn fn = []() -> EncodeTiledFn {
		void* p = nullptr;
		cudaDriverEntryPointQueryResult q;
		if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) return nullptr;
		if (q != cudaDriverEntryPointSuccess) return nullptr;
		return reinterpret_cast<EncodeTiledFn>(p);
	}();
	return fn;
}

// Encoding a map costs a few microseconds of host time; the mixer re-issues the same few (pointer, shape) pairs
// every step, so the most recent ones are kept.
struct TmapKey
{
	const void* base;
	uint64_t d[3], s[2];
	uint32_t box[2];
	int rank, f32, swizzle;
	bool operator==(const TmapKey& o) const { return std::memcmp(this, &o, sizeof(TmapKey)) == 0; }
};
struct TmapKeyHash
{
	size_t operator()(const TmapKey& k) const
	{
		const unsigned char* p = reinterpret_cast<const unsigned char*>(&k);
		size_t h = 1469598103934665603ull;  // FNV-1a
		for (size_t i = 0; i < sizeof(TmapKey); ++i) h = (h ^ p[i]) * 1099511628211ull;
		return h;
	}
};

static int cached_tmap(CUtensorMap* out, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_elems,
	const uint32_t* box01, bool f32 = false, bool swizzle128 = true)
{
	static std::mutex mu;
	static std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> cache;
	TmapKey key;
	std::memset(&key, 0, sizeof(key));  // padding bytes take part in the comparison
	key.base = base;
	key.rank = rank;
	for (int i = 0; i < rank; ++i) key.d[i] = dims[i];
	for (int i = 0; i + 1 < rank; ++i) key.s[i] = strides_elems[i];
	key.box[0] = box01[0];
	key.box[1] = box01[1];
	key.f32 = f32 ? 1 : 0;
	key.swizzle = swizzle128 ? 1 : 0;
	{
		std::lock_guard<std::mutex> lk(mu);
		auto it = cache.find(key);
		if (it != cache.end())
		{
			std::memcpy(out, &it->second, sizeof(CUtensorMap));
			return B200_OK;
		}
	}
	EncodeTiledFn fn = get_encode_fn();
	if (!fn) return B200_ERR_CUDA;
	cuuint64_t gd[3] = { 1, 1, 1 }, gs[2] = { 0, 0 };
	cuuint32_t bx[3] = { 1, 1, 1 }, es[3] = { 1, 1, 1 };
	for (int i = 0; i < rank; ++i) gd[i] = dims[i];
	for (int i = 0; i + 1 < rank; ++i) gs[i] = strides_elems[i] * (f32 ? sizeof(float) : sizeof(__half));
	bx[0] = box01[0];
	bx[1] = box01[1];
	const CUresult r = fn(out, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, static_cast<cuuint32_t>(rank),
		const_cast<void*>(base), gd, gs, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
		swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
		CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
	if (r != CUDA_SUCCESS)
	{
		g_last_cuda_error = static_cast<int>(r);
		return B200_ERR_CUDA;
	}
	std::lock_guard<std::mutex> lk(mu);
	if (cache.size() > 512) cache.clear();
	cache.emplace(key, *out);
	return B200_OK;
}

int tmap_2d_f16(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld_elems, uint32_t box_cols,
	uint32_t box_rows)
{
	const uint64_t dims[2] = { cols, rows };
	const uint64_t strides[1] = { ld_elems };
	const uint32_t box[2] = { box_cols, box_rows };
	return cached_tmap(out, base, 2, dims, strides, box);
}

int tmap_3d_f16(CUtensorMap* out, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t s1_elems, uint64_t s2_elems,
	uint32_t box0, uint32_t box1)
{
	const uint64_t dims[3] = { d0, d1, d2 };
	const uint64_t strides[2] = { s1_elems, s2_elems };
	const uint32_t box[2] = { box0, box1 };
	return cached_tmap(out, base, 3, dims, strides, box);
}

int tmap_3d_f16_linear(CUtensorMap* out, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t s1_elems,
	uint64_t s2_elems, uint32_t box0, uint32_t box1)
{
	const uint64_t dims[3] = { d0, d1, d2 };
	const uint64_t strides[2] = { s1_elems, s2_elems };
	const uint32_t box[2] = { box0, box1 };
	return cached_tmap(out, base, 3, dims, strides, box, false, false);
}

int tmap_3d_f32(CUtensorMap* out, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t s1_elems, uint64_t s2_elems,
	uint32_t box0, uint32_t box1)
{
	const uint64_t dims[3] = { d0, d1, d2 };
	const uint64_t strides[2] = { s1_elems, s2_elems };
	const uint32_t box[2] = { box0, box1 };
	return cached_tmap(out, base, 3, dims, strides, box, true, true);
}

int tmap_2d_f32_linear(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld_elems, uint32_t box_cols,
	uint32_t box_rows)
{
	const uint64_t dims[2] = { cols, rows };
	const uint64_t strides[1] = { ld_elems };
	const uint32_t box[2] = { box_cols, box_rows };
	return cached_tmap(out, base, 2, dims, strides, box, true, false);
}

}  // namespace b200
