// Shared declarations of the SSD chunked-scan stages (prefill).
//
// Stage structure follows mamba_chunk_scan_combined_ref (scripts/zamba2/mamba_chunk_scan_comb.py:167-215):
//   1. dt / cumsum     : dt = softplus(dt_raw + dt_bias), dA = dt*A, in-chunk inclusive cumsum      (:32-48)
//   2. chunk state     : states[b,c,h,p,n] = sum_l B[l,n] exp(dAcs[last]-dAcs[l]) dt[l] x[l,p]      (:51-80)
//   3. state passing   : running state across chunks; states[c] is replaced by the state BEFORE c   (:83-106)
//   4. chunk scan      : y = (C.B^T o decay o causal).(dt x) + exp(dAcs) C.prev^T + D x            (:109-160)
// Workspace layout: dt[b,H,nc,Q] f32 | dAcs[b,H,nc,Q] f32 | colf[b,H,nc,Q] f32 | states[b,nc,H,P,N] f32 | prev16[b,nc,H,P,N] f16
// colf[l] = exp(dAcs[end of l's 64-block] - dAcs[l]) * dt[l]: the column factor of the decay for score blocks that lie
// entirely below the diagonal, where exp(dAcs[l]-dAcs[s]) = exp(dAcs[l]-dAcs[end]) * exp(dAcs[end]-dAcs[s]) with both exponents <= 0.
// (prev16: the state before each chunk rounded to f16, the tensor-core operand of stage 4; the reference rounds the
// passed states to the activation dtype as well, scripts/zamba2/mamba_chunk_scan_comb.py:211).
#pragma once
#include "common.cuh"

namespace b200 {

struct SsdDims
{
	int64_t batch, seqlen;
	int H, P, G, N, Q, nchunks;
};

struct SsdWorkspace
{
	float* dt;
	float* dacs;
	float* colf;
	float* states;
	__half* prev16;
	size_t bytes;
};

inline SsdWorkspace ssd_carve(void* base, const SsdDims& d)
{
	SsdWorkspace w;
	const size_t n_dt = static_cast<size_t>(d.batch) * d.H * d.nchunks * d.Q;
	const size_t n_st = static_cast<size_t>(d.batch) * d.nchunks * d.H * d.P * d.N;
	const size_t o1 = align_up(n_dt * sizeof(float), 256);
	const size_t oc = o1 + align_up(n_dt * sizeof(float), 256);
	const size_t o2 = oc + align_up(n_dt * sizeof(float), 256);
	char* p = static_cast<char*>(base);
	w.dt = reinterpret_cast<float*>(p);
	w.dacs = reinterpret_cast<float*>(p + o1);
	w.colf = reinterpret_cast<float*>(p + oc);
	w.states = reinterpret_cast<float*>(p + o2);
	const size_t o3 = o2 + align_up(n_st * sizeof(float), 256);
	w.prev16 = reinterpret_cast<__half*>(p + o3);
	w.bytes = o3 + align_up(n_st * sizeof(__half), 256);
	return w;
}

// Stage launchers. T is the activation storage type.
template <typename T>
int ssd_dt_cumsum(const T* dt, int64_t dts, const float* A, int a_is_log, const float* dt_bias, int dt_softplus,
	const SsdDims& d, const SsdWorkspace& w, cudaStream_t st);

template <typename T>
int ssd_chunk_state_simt(const T* x, int64_t xs, const T* Bm, int64_t bs, const SsdDims& d, const SsdWorkspace& w, cudaStream_t st);

// write_prev16: also store the f16 copy of the state before each chunk (needed by the tensor-core chunk scan).
int ssd_state_passing(const float* initial_states, float* final_states, bool write_prev16, const SsdDims& d, const SsdWorkspace& w,
	cudaStream_t st, bool write_prev = true);
// log of the total decay of the segment per (batch, head), from the dt stage's results
int ssd_segment_logdecay(float* out, const SsdDims& d, const SsdWorkspace& w, cudaStream_t st);

// Tensor-core stages (f16 activations; shapes accepted by ssd_tc_supported).
bool ssd_tc_supported(const SsdDims& d, const void* x, int64_t xs, const void* Bm, int64_t bs, const void* Cm, int64_t cs, const void* y,
	int64_t ys);
int ssd_chunk_state_tc(const __half* x, int64_t xs, const __half* Bm, int64_t bs, const SsdDims& d, const SsdWorkspace& w, cudaStream_t st);
int ssd_chunk_scan_tc(const __half* x, int64_t xs, const __half* Bm, int64_t bs, const __half* Cm, int64_t cs, const float* D, __half* y,
	int64_t ys, const SsdDims& d, const SsdWorkspace& w, cudaStream_t st);

// The whole scan after the dt stage as one kernel (ssd_fused.cu): chunk states, state passing and chunk scan without the
// per-chunk states ever reaching HBM. `supported`: shapes and alignments it covers; `preferred`: whether it is expected to beat
// the staged kernels for this problem size (B200_SSD_FUSED=1 / 0 in the environment forces the answer).
bool ssd_fused_supported(const SsdDims& d, const void* x, int64_t xs, const void* Bm, int64_t bs, const void* Cm, int64_t cs, const void* y,
	int64_t ys, const float* init, const float* fin);
bool ssd_fused_preferred(const SsdDims& d);
int ssd_fused_tc(const __half* x, int64_t xs, const __half* Bm, int64_t bs, const __half* Cm, int64_t cs, const float* D,
	const float* init, __half* y, int64_t ys, float* fin, const SsdDims& d, const SsdWorkspace& w, cudaStream_t st);

// The one-kernel scan over a packed batch of sequences (see ssd_fused.cu).
bool ssd_fused_varlen_supported(int64_t total_tokens, int64_t nseq, int H, int P, int G, int N, const void* x, int64_t xs, const void* Bm,
	int64_t bs, const void* Cm, int64_t cs, const void* y, int64_t ys, const float* init, const float* fin);
int ssd_fused_varlen_tc(const __half* x, int64_t xs, const __half* Bm, int64_t bs, const __half* Cm, int64_t cs, const float* D,
	const float* init, __half* y, int64_t ys, float* fin, int64_t total_tokens, int64_t nseq, int H, int G, const float* dt_rows,
	const float* dacs_rows, const int* cu, const int* coff, int nblk, cudaStream_t st);

template <typename T>
int ssd_chunk_scan_simt(const T* x, int64_t xs, const T* Bm, int64_t bs, const T* Cm, int64_t cs, const float* D, T* y, int64_t ys,
	const SsdDims& d, const SsdWorkspace& w, cudaStream_t st);

}  // namespace b200
