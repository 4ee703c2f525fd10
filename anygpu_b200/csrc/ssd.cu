// C entry point of the SSD chunked selective scan: validates, carves the workspace and runs the four stages.
#include "ssd_common.cuh"

namespace b200 {

// The scan in parts. kSsdStageDt: softplus and in-chunk cumulative sums (needs dt only; the prefill mixer runs it inside its
// conv1d launch). kSsdStageStates: per-chunk states from x and B. kSsdStageSummary: the segment's state for a zero incoming
// state (written to `fin`) without touching the chunk states: what a GPU that holds one segment of a sequence sends on.
// kSsdStagePass: state passing from `init` and the chunk scan. A plain call runs Dt | States | Pass.
constexpr int kSsdStageDt = 1, kSsdStageStates = 2, kSsdStagePass = 4, kSsdStageSummary = 8;

template <typename T>
static int run_simt(const void* x, int64_t xs, const void* dt, int64_t dts, const float* A, int a_is_log, const void* Bm, int64_t bs,
	const void* Cm, int64_t cs, const float* D, const float* dt_bias, const float* init, void* y, int64_t ys, float* fin,
	const SsdDims& d, const SsdWorkspace& w, cudaStream_t st, int dt_softplus, int stages)
{
	int rc = B200_OK;
	if (stages & kSsdStageDt) rc = ssd_dt_cumsum<T>(static_cast<const T*>(dt), dts, A, a_is_log, dt_bias, dt_softplus, d, w, st);
	if (rc) return rc;
	if (stages & kSsdStageStates) rc = ssd_chunk_state_simt<T>(static_cast<const T*>(x), xs, static_cast<const T*>(Bm), bs, d, w, st);
	if (rc) return rc;
	if (stages & kSsdStageSummary) rc = ssd_state_passing(nullptr, fin, false, d, w, st, false);
	if (rc || !(stages & kSsdStagePass)) return rc;
	rc = ssd_state_passing(init, fin, false, d, w, st);
	if (rc) return rc;
	return ssd_chunk_scan_simt<T>(static_cast<const T*>(x), xs, static_cast<const T*>(Bm), bs, static_cast<const T*>(Cm), cs, D,
		static_cast<T*>(y), ys, d, w, st);
}

// f16 activations on the tensor cores: the two contractions run as tcgen05 kernels.
static int run_tc(const void* x, int64_t xs, const void* dt, int64_t dts, const float* A, int a_is_log, const void* Bm, int64_t bs,
	const void* Cm, int64_t cs, const float* D, const float* dt_bias, const float* init, void* y, int64_t ys, float* fin,
	const SsdDims& d, const SsdWorkspace& w, cudaStream_t st, int dt_softplus, int stages)
{
	const __half* xh = static_cast<const __half*>(x);
	const __half* bh = static_cast<const __half*>(Bm);
	const __half* ch = static_cast<const __half*>(Cm);
	int rc = B200_OK;
	if (stages & kSsdStageDt) rc = ssd_dt_cumsum<__half>(static_cast<const __half*>(dt), dts, A, a_is_log, dt_bias, dt_softplus, d, w, st);
	if (rc) return rc;
	// a whole scan (no stage left to another call): one kernel where it covers the shape and the problem is large enough in
	// (batch x heads) for it
	if ((stages & (kSsdStageStates | kSsdStagePass | kSsdStageSummary)) == (kSsdStageStates | kSsdStagePass) &&
		ssd_fused_supported(d, x, xs, Bm, bs, Cm, cs, y, ys, init, fin) && ssd_fused_preferred(d))
		return ssd_fused_tc(xh, xs, bh, bs, ch, cs, D, init, static_cast<__half*>(y), ys, fin, d, w, st);
	if (stages & kSsdStageStates) rc = ssd_chunk_state_tc(xh, xs, bh, bs, d, w, st);
	if (rc) return rc;
	if (stages & kSsdStageSummary) rc = ssd_state_passing(nullptr, fin, true, d, w, st, false);
	if (rc || !(stages & kSsdStagePass)) return rc;
	rc = ssd_state_passing(init, fin, true, d, w, st);
	if (rc) return rc;
	return ssd_chunk_scan_tc(xh, xs, bh, bs, ch, cs, D, static_cast<__half*>(y), ys, d, w, st);
}

}  // namespace b200

using namespace b200;

extern "C" size_t b200_mamba_chunk_scan_combined_workspace_bytes(int64_t batch, int64_t seqlen, int64_t H, int64_t P, int64_t G,
	int64_t N, int64_t chunk)
{
	if (batch <= 0 || seqlen <= 0 || H <= 0 || P <= 0 || G <= 0 || N <= 0 || chunk <= 0) return 0;
	SsdDims d{ batch, seqlen, static_cast<int>(H), static_cast<int>(P), static_cast<int>(G), static_cast<int>(N),
		static_cast<int>(chunk), static_cast<int>(cdiv(seqlen, chunk)) };
	return ssd_carve(nullptr, d).bytes;
}

namespace b200 {
int ssd_combined_stages(int dtype, const void* x, int64_t x_stride, const void* dt, int64_t dt_stride,
	const float* A, int a_is_log, const void* B, int64_t B_stride, const void* C, int64_t C_stride,
	const float* D, const float* dt_bias, const float* initial_states,
	void* y, int64_t y_stride, float* final_states,
	int64_t batch, int64_t seqlen, int64_t H, int64_t P, int64_t G, int64_t N, int64_t chunk, int dt_softplus,
	void* workspace, size_t workspace_bytes, void* stream, int stages)
{
	if (!x || !dt || !A || !B || !C || !y) return B200_ERR_NULL;
	if (batch < 0 || seqlen < 0 || H <= 0 || P <= 0 || G <= 0 || N <= 0 || chunk <= 0 || H % G != 0) return B200_ERR_BAD_SHAPE;
	if (chunk > 256) return B200_ERR_UNSUPPORTED;
	if (x_stride < H * P || y_stride < H * P || dt_stride < H || B_stride < G * N || C_stride < G * N) return B200_ERR_BAD_SHAPE;
	if (dtype != B200_F16 && dtype != B200_F32) return B200_ERR_UNSUPPORTED;
	// the mixer always applies softplus (scripts/zamba2/mamba_chunk_scan_comb.py:44-45)
	if (dt_softplus != B200_DT_SOFTPLUS && dt_softplus != B200_DT_SOFTPLUS_EXACT) return B200_ERR_UNSUPPORTED;
	if (batch == 0 || seqlen == 0) return B200_OK;
	if (batch * cdiv(seqlen, chunk) * H > 0x7fffffffLL) return B200_ERR_UNSUPPORTED;
	SsdDims d{ batch, seqlen, static_cast<int>(H), static_cast<int>(P), static_cast<int>(G), static_cast<int>(N),
		static_cast<int>(chunk), static_cast<int>(cdiv(seqlen, chunk)) };
	if (!workspace) return B200_ERR_WORKSPACE;
	if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return B200_ERR_MISALIGNED;
	const SsdWorkspace w = ssd_carve(workspace, d);
	if (workspace_bytes < w.bytes) return B200_ERR_WORKSPACE;
	cudaStream_t st = static_cast<cudaStream_t>(stream);
	if (dtype == B200_F16 && ssd_tc_supported(d, x, x_stride, B, B_stride, C, C_stride, y, y_stride))
		return run_tc(x, x_stride, dt, dt_stride, A, a_is_log, B, B_stride, C, C_stride, D, dt_bias, initial_states, y, y_stride,
			final_states, d, w, st, dt_softplus, stages);
	if (dtype == B200_F16)
		return run_simt<__half>(x, x_stride, dt, dt_stride, A, a_is_log, B, B_stride, C, C_stride, D, dt_bias, initial_states, y,
			y_stride, final_states, d, w, st, dt_softplus, stages);
	return run_simt<float>(x, x_stride, dt, dt_stride, A, a_is_log, B, B_stride, C, C_stride, D, dt_bias, initial_states, y,
		y_stride, final_states, d, w, st, dt_softplus, stages);
}

int ssd_segment_logdecay_of(float* out, int64_t batch, int64_t seqlen, int64_t H, int64_t P, int64_t G, int64_t N, int64_t chunk,
	void* workspace, cudaStream_t st)
{
	const SsdDims d{ batch, seqlen, static_cast<int>(H), static_cast<int>(P), static_cast<int>(G), static_cast<int>(N),
		static_cast<int>(chunk), static_cast<int>(cdiv(seqlen, chunk)) };
	return ssd_segment_logdecay(out, d, ssd_carve(workspace, d), st);
}
}  // namespace b200

extern "C" int b200_mamba_chunk_scan_combined(int dtype, const void* x, int64_t x_stride, const void* dt, int64_t dt_stride,
	const float* A, int a_is_log, const void* B, int64_t B_stride, const void* C, int64_t C_stride,
	const float* D, const float* dt_bias, const float* initial_states,
	void* y, int64_t y_stride, float* final_states,
	int64_t batch, int64_t seqlen, int64_t H, int64_t P, int64_t G, int64_t N, int64_t chunk, int dt_softplus,
	void* workspace, size_t workspace_bytes, void* stream)
{
	return ssd_combined_stages(dtype, x, x_stride, dt, dt_stride, A, a_is_log, B, B_stride, C, C_stride, D, dt_bias, initial_states, y,
		y_stride, final_states, batch, seqlen, H, P, G, N, chunk, dt_softplus, workspace, workspace_bytes, stream,
		kSsdStageDt | kSsdStageStates | kSsdStagePass);
}
