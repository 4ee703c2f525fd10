// The Mamba2 mixer of a Zamba2 block, composed from the operators of this library with every slice of the
// in_proj output (z | xBC | dt) and of the conv output (x | B | C) consumed in place through row strides:
//   prefill: in_proj GEMM -> causal conv1d+SiLU (token-major) -> SSD chunked scan -> gated RMSNorm -> out_proj GEMM
//   decode : in_proj GEMM -> conv_state update -> ssm_state recurrence -> gated RMSNorm -> out_proj GEMM
// Six to eight launches on one stream, no allocation, no host synchronisation.
#include <mutex>
#include <vector>

#include "common.cuh"

namespace b200 {

struct MixerDims
{
	int64_t conv_dim, d_in_proj;
	int64_t ldz;  // row stride of the in_proj output inside the workspaces: d_in_proj rounded up to 8 elements, so that its rows (and
	              // the z | xBC | dt slices, whose offsets are multiples of 8 for headdim and d_state multiples of 8) stay 16-byte aligned
	size_t esz;
};

static bool dims_ok(const b200_mamba2_config* c, int dtype, MixerDims* m)
{
	if (!c) return false;
	if (c->d_model <= 0 || c->d_inner <= 0 || c->nheads <= 0 || c->headdim <= 0 || c->d_state <= 0 || c->ngroups <= 0 ||
		c->d_conv < 1 || c->d_conv > 4 || c->chunk <= 0)
		return false;
	if (c->nheads * c->headdim != c->d_inner || c->nheads % c->ngroups != 0) return false;
	if (c->norm_group_size != 0 && c->d_inner % c->norm_group_size != 0) return false;
	if (dtype != B200_F16 && dtype != B200_F32) return false;
	m->conv_dim = c->d_inner + 2 * c->ngroups * c->d_state;
	m->d_in_proj = 2 * c->d_inner + 2 * c->ngroups * c->d_state + c->nheads;
	m->ldz = (m->d_in_proj + 7) / 8 * 8;
	m->esz = dtype == B200_F16 ? 2 : 4;
	return true;
}

// conv1d + the scan's dt stage in one launch (conv_dt_fused.cu), and the scan without / with chosen stages (ssd.cu)
constexpr int kSsdStageDt = 1, kSsdStageStates = 2, kSsdStagePass = 4, kSsdStageSummary = 8;
bool conv_dt_fused_applies(int dtype, const void* x, int64_t xs, const void* y, int64_t ys, const void* w, const void* bias, int64_t batch,
	int64_t seqlen, int64_t dims, int width);
int conv1d_tokens_with_scan_dt(int dtype, const void* x, int64_t xs, const void* w, const void* bias, void* y, int64_t ys,
	const void* init, void* fin, int64_t batch, int64_t seqlen, int64_t dims, int width, const void* dt, int64_t dts, const float* A,
	int a_is_log, const float* dt_bias, int dt_softplus, int64_t H, int64_t P, int64_t G, int64_t N, int64_t chunk, void* ssd_workspace,
	size_t ssd_workspace_bytes, cudaStream_t st);
int ssd_combined_stages(int dtype, const void* x, int64_t x_stride, const void* dt, int64_t dt_stride,
	const float* A, int a_is_log, const void* B, int64_t B_stride, const void* C, int64_t C_stride,
	const float* D, const float* dt_bias, const float* initial_states,
	void* y, int64_t y_stride, float* final_states,
	int64_t batch, int64_t seqlen, int64_t H, int64_t P, int64_t G, int64_t N, int64_t chunk, int dt_softplus,
	void* workspace, size_t workspace_bytes, void* stream, int stages);

// packed variable-length batches in a fixed number of launches (varlen.cu)
bool mixer_varlen_fused_applies(int dtype, const void* xbc_in, int64_t xs, const void* xbc, int64_t conv_dim, const void* conv_w,
	const void* conv_b, int width, int64_t total_tokens, int64_t nseq, int64_t H, int64_t P, int64_t G, int64_t N, const void* y, int64_t ys,
	const float* init, const float* fin);
int mixer_conv_ssd_varlen_f16(const void* xbc_in, int64_t xs, const void* conv_w, const void* conv_b, int width, void* xbc, int64_t conv_dim,
	void* conv_state_out, const void* dt, int64_t dts, const float* A_log, const float* dt_bias, const float* D, const float* init, void* y,
	int64_t ys, float* fin, const int64_t* cu_host, int64_t nseq, int64_t H, int64_t P, int64_t G, int64_t N, void* scratch,
	size_t scratch_bytes, cudaStream_t st);

int ssd_segment_logdecay_of(float* out, int64_t batch, int64_t seqlen, int64_t H, int64_t P, int64_t G, int64_t N, int64_t chunk,
	void* workspace, cudaStream_t st);
int ssd_segment_prefix(const float* seg_states, const float* seg_logdecay, int nseg, int64_t batch, int64_t H, int64_t P, int64_t N,
	float* state_in, cudaStream_t st);

int linear_f16_residual(const void* x, int64_t ldx, const void* w, int w_layout, void* y, int64_t ldy, int64_t M, int64_t K, int64_t N,
	const void* residual, int64_t ldr, cudaStream_t st);
int gated_rmsnorm_last_use(int dtype, const void* x, int64_t xs, const void* z, int64_t zs, const void* w, void* y, int64_t ys,
	int64_t rows, int64_t d, int64_t group_size, float eps, cudaStream_t st);

// fused decode stages (gemm_decode.cu, ssm_update.cu)
bool decode_linear_applies(int dtype, int64_t M, int64_t K, int64_t N);
size_t decode_linear_partial_bytes(int64_t M, int64_t K, int64_t N);
int decode_in_proj_conv(const void* x, int64_t ldx, const void* w, int w_layout, void* zx, int64_t ldz, int64_t M, int64_t K, int64_t N,
	int64_t conv_lo, int64_t conv_dim, int conv_width, void* conv_state, const void* conv_w, const void* conv_b, void* xbc, float* part,
	cudaStream_t st);
int decode_out_proj_scale(const void* x, int64_t ldx, const void* w, int w_layout, void* out, int64_t ldo, int64_t M, int64_t K, int64_t N,
	const float* sumsq, int nsumsq, int64_t norm_dim, float eps, float* part, cudaStream_t st, const void* residual, int64_t ldr);
bool ssm_update_gated_applies(int64_t H, int64_t P, int64_t N, int64_t G);
int ssm_update_gated_partials();
int ssm_update_gated_f16(float* state, const void* x, int64_t xs, const void* dt, int64_t dts, const float* A, int a_is_log, const void* Bm,
	int64_t bs, const void* Cm, int64_t cs, const float* D, const float* dt_bias, void* y, int64_t ys, const void* z, int64_t zs,
	const void* norm_w, float* sumsq, int64_t batch, int64_t H, int64_t P, int64_t G, int64_t N, int dt_softplus, cudaStream_t st);

// ---- optional per-stage timing of the prefill mixer (CUDA events on the caller's stream) -------------------------
constexpr int kStages = 5;       // in_proj, conv1d, ssd, gated_rmsnorm, out_proj
constexpr int kTimingSlots = 256;  // mixer calls recorded between two collects

struct StageTiming
{
	bool enabled = false;
	int last_stage = kStages;  // marks 0 .. last_stage are recorded: kStages = every stage, 1 = the first stage (in_proj) only
	int every = 1;             // every n-th call is recorded
	int seen = 0;              // calls since enable
	int calls = 0;
	cudaEvent_t ev[kTimingSlots][kStages + 1] = {};
	bool created = false;
};
static StageTiming g_timing;

static void stage_mark(int stage, cudaStream_t st)
{
	if (g_timing.enabled && stage <= g_timing.last_stage && g_timing.seen % g_timing.every == 0 && g_timing.calls < kTimingSlots)
	{
		// in a stream that is being captured an ordinary record would only become an edge of the graph; the external form makes a
		// node that records the event on every replay, so a harness can time the stages of a replayed graph
		cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
		if (cudaStreamIsCapturing(st, &cap) == cudaSuccess && cap == cudaStreamCaptureStatusActive)
			cudaEventRecordWithFlags(g_timing.ev[g_timing.calls][stage], st, cudaEventRecordExternal);
		else
			cudaEventRecord(g_timing.ev[g_timing.calls][stage], st);
	}
}

struct PrefillWs
{
	char* zxbcdt;
	char* xbc;
	char* y;
	char* ssd;
	size_t ssd_bytes;
	size_t bytes;
};

static PrefillWs carve_prefill(void* base, const b200_mamba2_config* c, const MixerDims& m, int64_t batch, int64_t seqlen)
{
	PrefillWs w;
	const size_t T = static_cast<size_t>(batch) * seqlen;
	char* p = static_cast<char*>(base);
	size_t off = 0;
	w.zxbcdt = p + off; off += align_up(T * m.ldz * m.esz, 256);
	w.xbc = p + off; off += align_up(T * m.conv_dim * m.esz, 256);
	w.y = p + off; off += align_up(T * c->d_inner * m.esz, 256);
	w.ssd = p + off;
	w.ssd_bytes = b200_mamba_chunk_scan_combined_workspace_bytes(batch, seqlen, c->nheads, c->headdim, c->ngroups, c->d_state, c->chunk);
	off += w.ssd_bytes;
	w.bytes = off;
	return w;
}


// out += residual, row by row (the paths whose projection has no fused residual: fp32 tensors, unaligned shapes)
template <typename T>
__global__ void __launch_bounds__(256) residual_add_kernel(T* __restrict__ out, int64_t ldo, const T* __restrict__ res, int64_t ldr,
	int64_t rows, int cols)
{
	const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
	if (i >= rows * cols) return;
	const int64_t r = i / cols;
	const int c = static_cast<int>(i - r * cols);
	stf(out + r * ldo + c, ldf(out + r * ldo + c) + ldf(res + r * ldr + c));
}

static int residual_add(int dtype, void* out, int64_t ldo, const void* res, int64_t ldr, int64_t rows, int64_t cols, cudaStream_t st)
{
	const int64_t blocks = cdiv(rows * cols, 256);
	if (blocks > 0x7fffffffLL) return B200_ERR_UNSUPPORTED;
	if (dtype == B200_F16)
		residual_add_kernel<__half><<<static_cast<unsigned>(blocks), 256, 0, st>>>(static_cast<__half*>(out), ldo,
			static_cast<const __half*>(res), ldr, rows, static_cast<int>(cols));
	else
		residual_add_kernel<float><<<static_cast<unsigned>(blocks), 256, 0, st>>>(static_cast<float*>(out), ldo,
			static_cast<const float*>(res), ldr, rows, static_cast<int>(cols));
	B200_LAUNCH_CHECK();
	return B200_OK;
}

// out = y . W_out (+ residual): the projection that ends the mixer; the residual of the layer around it rides in the epilogue
// of the f16 tensor-core GEMM; where that kernel cannot take the shape (fp32 tensors, sizes or strides off the 8-element grid,
// which b200_linear runs on its SIMT kernel) it is added by a second kernel.
static int out_proj_residual(int dtype, const void* y, int64_t ldy, const void* w, int layout, void* out, int64_t ldo, int64_t T,
	int64_t K, int64_t N, const void* residual, int64_t ldr, cudaStream_t st)
{
	if (residual && dtype == B200_F16 && K % 8 == 0 && N % 8 == 0 && ldr % 8 == 0 && aligned16(residual))
		return linear_f16_residual(y, ldy, w, layout, out, ldo, T, K, N, residual, ldr, st);
	const int rc = b200_linear(dtype, y, ldy, w, layout, out, ldo, T, K, N, st);
	if (rc || !residual) return rc;
	return residual_add(dtype, out, ldo, residual, ldr, T, N, st);
}
}  // namespace b200

using namespace b200;

extern "C" size_t b200_mamba2_mixer_prefill_workspace_bytes(const b200_mamba2_config* cfg, int dtype, int64_t batch, int64_t seqlen)
{
	MixerDims m;
	if (!dims_ok(cfg, dtype, &m) || batch <= 0 || seqlen <= 0) return 0;
	return carve_prefill(nullptr, cfg, m, batch, seqlen).bytes;
}

// The stages between the two projections for `batch` sequences of `seqlen` tokens whose projected rows start at `zxbcdt`:
// conv1d + SiLU over the xBC columns (with the scan's dt stage in the same launch where that applies), then the chunked scan.
static int mixer_conv_ssd(int dtype, const b200_mamba2_config* cfg, const b200_mamba2_weights* w, const MixerDims& m, const char* zxbcdt,
	char* xbc, char* y, char* ssd, size_t ssd_bytes, int64_t batch, int64_t seqlen, const float* initial_states, const void* conv_state_in,
	void* conv_state_out, float* ssm_state_out, cudaStream_t st, bool mark)
{
	const int64_t d_inner = cfg->d_inner, GN = cfg->ngroups * cfg->d_state;
	const size_t e = m.esz;
	const char* dtp = zxbcdt + (d_inner + m.conv_dim) * e;
	const bool dt_in_conv = conv_dt_fused_applies(dtype, zxbcdt + d_inner * e, m.ldz, xbc, m.conv_dim, w->conv1d_weight, w->conv1d_bias, batch, seqlen, m.conv_dim,
		static_cast<int>(cfg->d_conv)) && cfg->chunk <= 256 && batch * cdiv(seqlen, cfg->chunk) * cfg->nheads <= 0x7fffffffLL;
	int rc;
	if (dt_in_conv)
		rc = conv1d_tokens_with_scan_dt(dtype, zxbcdt + d_inner * e, m.ldz, w->conv1d_weight, w->conv1d_bias, xbc, m.conv_dim,
			conv_state_in, conv_state_out, batch, seqlen, m.conv_dim, static_cast<int>(cfg->d_conv), dtp, m.ldz, w->A_log, 1, w->dt_bias,
			B200_DT_SOFTPLUS_EXACT, cfg->nheads, cfg->headdim, cfg->ngroups, cfg->d_state, cfg->chunk, ssd, ssd_bytes, st);
	else
		rc = b200_causal_conv1d_tokens(dtype, zxbcdt + d_inner * e, m.ldz, w->conv1d_weight, w->conv1d_bias, xbc, m.conv_dim,
			conv_state_in, conv_state_out, batch, seqlen, m.conv_dim, static_cast<int>(cfg->d_conv), st);
	if (rc) return rc;
	if (mark) stage_mark(2, st);
	return ssd_combined_stages(dtype, xbc, m.conv_dim, dtp, m.ldz, w->A_log, 1, xbc + d_inner * e, m.conv_dim,
		xbc + (d_inner + GN) * e, m.conv_dim, w->D, w->dt_bias, initial_states, y, d_inner, ssm_state_out, batch, seqlen, cfg->nheads,
		cfg->headdim, cfg->ngroups, cfg->d_state, cfg->chunk, B200_DT_SOFTPLUS_EXACT, ssd, ssd_bytes, st,
		(dt_in_conv ? 0 : kSsdStageDt) | kSsdStageStates | kSsdStagePass);
}

// The prefill mixer; `residual` [T, >= d_model] (or nullptr) is added to the result (may alias `out`).
static int mixer_prefill_impl(int dtype, const b200_mamba2_config* cfg, const b200_mamba2_weights* w,
	const void* u, void* out, int64_t batch, int64_t seqlen,
	const float* initial_states, void* conv_state_out, float* ssm_state_out,
	void* workspace, size_t workspace_bytes, void* stream, const void* residual, int64_t ldr, const void* conv_state_in = nullptr)
{
	if (!cfg || !w || !u || !out) return B200_ERR_NULL;
	if (!w->in_proj_weight || !w->conv1d_weight || !w->conv1d_bias || !w->dt_bias || !w->A_log || !w->D || !w->norm_weight ||
		!w->out_proj_weight)
		return B200_ERR_NULL;
	MixerDims m;
	if (!dims_ok(cfg, dtype, &m) || batch < 0 || seqlen < 0) return B200_ERR_BAD_SHAPE;
	if (batch == 0 || seqlen == 0) return B200_OK;
	if (!workspace) return B200_ERR_WORKSPACE;
	if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return B200_ERR_MISALIGNED;
	const PrefillWs ws = carve_prefill(workspace, cfg, m, batch, seqlen);
	if (workspace_bytes < ws.bytes) return B200_ERR_WORKSPACE;

	const int64_t T = batch * seqlen;
	const int64_t d_inner = cfg->d_inner;
	cudaStream_t st = static_cast<cudaStream_t>(stream);
	stage_mark(0, st);
	int rc = b200_linear(dtype, u, cfg->d_model, w->in_proj_weight, w->in_proj_layout, ws.zxbcdt, m.ldz, T, cfg->d_model,
		m.d_in_proj, stream);
	if (rc) return rc;
	stage_mark(1, st);
	rc = mixer_conv_ssd(dtype, cfg, w, m, ws.zxbcdt, ws.xbc, ws.y, ws.ssd, ws.ssd_bytes, batch, seqlen, initial_states, conv_state_in,
		conv_state_out, ssm_state_out, st, true);
	if (rc) return rc;
	stage_mark(3, st);
	rc = gated_rmsnorm_last_use(dtype, ws.y, d_inner, ws.zxbcdt, m.ldz, w->norm_weight, ws.y, d_inner, T, d_inner,
		cfg->norm_group_size, cfg->eps, st);
	if (rc) return rc;
	stage_mark(4, st);
	rc = out_proj_residual(dtype, ws.y, d_inner, w->out_proj_weight, w->out_proj_layout, out, cfg->d_model, T, d_inner, cfg->d_model,
		residual, ldr, st);
	if (rc) return rc;
	stage_mark(5, st);
	if (g_timing.enabled)
	{
		if (g_timing.seen % g_timing.every == 0 && g_timing.calls < kTimingSlots) ++g_timing.calls;
		++g_timing.seen;
	}
	return B200_OK;
}

extern "C" int b200_mamba2_mixer_prefill(int dtype, const b200_mamba2_config* cfg, const b200_mamba2_weights* w,
	const void* u, void* out, int64_t batch, int64_t seqlen,
	const float* initial_states, void* conv_state_out, float* ssm_state_out,
	void* workspace, size_t workspace_bytes, void* stream)
{
	return mixer_prefill_impl(dtype, cfg, w, u, out, batch, seqlen, initial_states, conv_state_out, ssm_state_out, workspace,
		workspace_bytes, stream, nullptr, 0);
}

extern "C" int b200_stage_timing_enable(int enable)
{
	if (enable && !g_timing.created)
	{
		for (int i = 0; i < kTimingSlots; ++i)
			for (int j = 0; j <= kStages; ++j) B200_CUDA_TRY(cudaEventCreate(&g_timing.ev[i][j]));
		g_timing.created = true;
	}
	g_timing.enabled = enable != 0;
	g_timing.last_stage = enable == 2 ? 1 : kStages;
	g_timing.every = enable == 2 ? 4 : 1;
	g_timing.seen = 0;
	g_timing.calls = 0;
	return B200_OK;
}

extern "C" int b200_stage_timing_collect(float* stage_ms, int* calls)
{
	if (!stage_ms || !calls) return B200_ERR_NULL;
	for (int j = 0; j < kStages; ++j) stage_ms[j] = 0.f;
	*calls = g_timing.calls;
	for (int i = 0; i < g_timing.calls; ++i)
	{
		B200_CUDA_TRY(cudaEventSynchronize(g_timing.ev[i][g_timing.last_stage]));
		for (int j = 0; j < g_timing.last_stage; ++j)
		{
			float ms = 0.f;
			B200_CUDA_TRY(cudaEventElapsedTime(&ms, g_timing.ev[i][j], g_timing.ev[i][j + 1]));
			stage_ms[j] += ms;
		}
	}
	g_timing.calls = 0;
	return B200_OK;
}

extern "C" size_t b200_mamba2_mixer_prefill_host_workspace_bytes(const b200_mamba2_config* cfg, int dtype, int64_t batch,
	int64_t seqlen)
{
	MixerDims m;
	if (!dims_ok(cfg, dtype, &m) || batch <= 0 || seqlen <= 0) return 0;
	const size_t io = align_up(static_cast<size_t>(batch) * seqlen * cfg->d_model * m.esz, 256);
	return 2 * io + carve_prefill(nullptr, cfg, m, batch, seqlen).bytes;
}

// Engines of the host-buffer entry point: one stream for host->device, one for the mixer, one for device->host, created
// once per device, plus per-sequence events. The three activities of consecutive sequences overlap:
//   copy-in(i+1)  ||  mixer(i)  ||  copy-out(i-1)
// The caller's stream only hands over to them at the start of a call and waits for the last copy-out at its end.
namespace b200 {
struct HostPipe
{
	cudaStream_t s_in = nullptr, s_comp = nullptr, s_out = nullptr;
	cudaEvent_t ev_start = nullptr, ev_end = nullptr;
	std::vector<cudaEvent_t> ev_in, ev_done, ev_out;  // per slice of sequences: copied in, mixer done, copied out
	// the call before this one on the device: where its staging tensors were, how it was cut into sequences, and its stream
	const void* last_ws = nullptr;
	int64_t last_batch = 0;
	size_t last_seq_bytes = 0;
	cudaStream_t last_stream = nullptr;
	int last_flags = 0;
};
static int host_pipe(HostPipe** out, int64_t nchunks)
{
	static HostPipe pipes[64];
	int dev = 0;
	B200_CUDA_TRY(cudaGetDevice(&dev));
	if (dev < 0 || dev >= 64) return B200_ERR_UNSUPPORTED;
	HostPipe& p = pipes[dev];
	if (!p.s_in)
	{
		B200_CUDA_TRY(cudaStreamCreateWithFlags(&p.s_in, cudaStreamNonBlocking));
		B200_CUDA_TRY(cudaStreamCreateWithFlags(&p.s_comp, cudaStreamNonBlocking));
		B200_CUDA_TRY(cudaStreamCreateWithFlags(&p.s_out, cudaStreamNonBlocking));
		B200_CUDA_TRY(cudaEventCreateWithFlags(&p.ev_start, cudaEventDisableTiming));
		B200_CUDA_TRY(cudaEventCreateWithFlags(&p.ev_end, cudaEventDisableTiming));
	}
	while (static_cast<int64_t>(p.ev_in.size()) < nchunks)
	{
		cudaEvent_t a, b, c;
		B200_CUDA_TRY(cudaEventCreateWithFlags(&a, cudaEventDisableTiming));
		B200_CUDA_TRY(cudaEventCreateWithFlags(&b, cudaEventDisableTiming));
		B200_CUDA_TRY(cudaEventCreateWithFlags(&c, cudaEventDisableTiming));
		p.ev_in.push_back(a);
		p.ev_done.push_back(b);
		p.ev_out.push_back(c);
	}
	*out = &p;
	return B200_OK;
}
}  // namespace b200

extern "C" int b200_mamba2_mixer_prefill_host_ex(int dtype, const b200_mamba2_config* cfg, const b200_mamba2_weights* w,
	const void* u_host, void* out_host, int64_t batch, int64_t seqlen,
	void* workspace, size_t workspace_bytes, void* stream, int flags)
{
	if (!cfg || !w || !u_host || !out_host) return B200_ERR_NULL;
	if (flags & ~B200_HOST_OVERLAP) return B200_ERR_UNSUPPORTED;
	MixerDims m;
	if (!dims_ok(cfg, dtype, &m) || batch < 0 || seqlen < 0) return B200_ERR_BAD_SHAPE;
	if (batch == 0 || seqlen == 0) return B200_OK;
	if (!workspace) return B200_ERR_WORKSPACE;
	if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return B200_ERR_MISALIGNED;
	const size_t io_bytes = static_cast<size_t>(batch) * seqlen * cfg->d_model * m.esz;
	const size_t io = align_up(io_bytes, 256);
	const size_t inner = carve_prefill(nullptr, cfg, m, batch, seqlen).bytes;
	if (workspace_bytes < 2 * io + inner) return B200_ERR_WORKSPACE;
	char* p = static_cast<char*>(workspace);
	char* u_dev = p;
	char* out_dev = p + io;
	cudaStream_t st = static_cast<cudaStream_t>(stream);

	// A pipeline step is a slice of whole sequences (they are independent through every stage of the mixer): one sequence by
	// default, which starts the compute soonest; with B200_HOST_OVERLAP enough sequences for ~4096 tokens (but at least two slices
	// per call), because there the loop's rate counts and a lone short sequence leaves the GPU underfilled (the scan walks a
	// sequence block by block whatever the batch). The copy streams and events are shared by all calls on a device: calls from
	// several host threads enqueue one after the other.
	int64_t per_slice = 1;
	if (flags & B200_HOST_OVERLAP)
	{
		per_slice = cdiv(4096, seqlen);
		if (per_slice > batch / 2) per_slice = batch / 2;
		if (per_slice < 1) per_slice = 1;
	}
	const int64_t nslices = cdiv(batch, per_slice);
	static std::mutex pipe_mutex;
	std::lock_guard<std::mutex> pipe_lock(pipe_mutex);
	HostPipe* hp = nullptr;
	int rc = host_pipe(&hp, nslices);
	if (rc) return rc;
	const size_t seq_bytes = static_cast<size_t>(seqlen) * cfg->d_model * m.esz;
	const size_t slice_bytes = static_cast<size_t>(per_slice) * seq_bytes;
	const char* uh = static_cast<const char*>(u_host);
	char* oh = static_cast<char*>(out_host);
	// What does the call wait for? By default for whatever the caller already queued on `stream` (which may be what fills u_host
	// or the weights), and that includes the copy-out of the call before this one. With B200_HOST_OVERLAP the caller vouches that
	// the call needs nothing queued on `stream` since the call before it; a call that repeats that one (same workspace, stream,
	// shape and flags) then only keeps off each staging slice while the earlier call still uses it: its copy-in of slice i waits
	// for the earlier mixer of slice i, its mixer of slice i for the earlier copy-out of slice i. Back-to-back calls so keep both
	// copy directions busy. Any other history, and a stream that is being captured into a graph, takes the default.
	cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
	B200_CUDA_TRY(cudaStreamIsCapturing(st, &capturing));
	const bool repeat = (flags & B200_HOST_OVERLAP) && capturing == cudaStreamCaptureStatusNone && hp->last_ws == workspace &&
		hp->last_batch == batch && hp->last_seq_bytes == seq_bytes && hp->last_stream == st && hp->last_flags == flags;
	if (!repeat)
	{
		B200_CUDA_TRY(cudaEventRecord(hp->ev_start, st));
		B200_CUDA_TRY(cudaStreamWaitEvent(hp->s_in, hp->ev_start, 0));
		B200_CUDA_TRY(cudaStreamWaitEvent(hp->s_comp, hp->ev_start, 0));
		B200_CUDA_TRY(cudaStreamWaitEvent(hp->s_out, hp->ev_start, 0));
	}
	auto bytes_of = [&](int64_t i) { return static_cast<size_t>((i + 1) * per_slice <= batch ? per_slice : batch - i * per_slice) * seq_bytes; };
	for (int64_t i = 0; i < nslices; ++i)
	{
		if (repeat) B200_CUDA_TRY(cudaStreamWaitEvent(hp->s_in, hp->ev_done[i], 0));  // recorded by the call before: its mixer of slice i
		B200_CUDA_TRY(cudaMemcpyAsync(u_dev + i * slice_bytes, uh + i * slice_bytes, bytes_of(i), cudaMemcpyHostToDevice, hp->s_in));
		B200_CUDA_TRY(cudaEventRecord(hp->ev_in[i], hp->s_in));
	}
	hp->last_ws = nullptr;  // an early return below leaves no history to build on
	for (int64_t i = 0; i < nslices; ++i)
	{
		B200_CUDA_TRY(cudaStreamWaitEvent(hp->s_comp, hp->ev_in[i], 0));
		if (repeat) B200_CUDA_TRY(cudaStreamWaitEvent(hp->s_comp, hp->ev_out[i], 0));  // the call before: its copy-out of slice i
		rc = b200_mamba2_mixer_prefill(dtype, cfg, w, u_dev + i * slice_bytes, out_dev + i * slice_bytes,
			static_cast<int64_t>(bytes_of(i) / seq_bytes), seqlen, nullptr, nullptr, nullptr, p + 2 * io, inner, hp->s_comp);
		if (rc) return rc;
		B200_CUDA_TRY(cudaEventRecord(hp->ev_done[i], hp->s_comp));
		B200_CUDA_TRY(cudaStreamWaitEvent(hp->s_out, hp->ev_done[i], 0));
		B200_CUDA_TRY(cudaMemcpyAsync(oh + i * slice_bytes, out_dev + i * slice_bytes, bytes_of(i), cudaMemcpyDeviceToHost, hp->s_out));
		B200_CUDA_TRY(cudaEventRecord(hp->ev_out[i], hp->s_out));
	}
	// work queued on `stream` after this call (and a synchronisation of `stream`) sees the finished output
	B200_CUDA_TRY(cudaEventRecord(hp->ev_end, hp->s_out));
	B200_CUDA_TRY(cudaStreamWaitEvent(st, hp->ev_end, 0));
	hp->last_ws = workspace;
	hp->last_batch = batch;
	hp->last_seq_bytes = seq_bytes;
	hp->last_stream = st;
	hp->last_flags = flags;
	return B200_OK;
}

extern "C" int b200_mamba2_mixer_prefill_host(int dtype, const b200_mamba2_config* cfg, const b200_mamba2_weights* w,
	const void* u_host, void* out_host, int64_t batch, int64_t seqlen,
	void* workspace, size_t workspace_bytes, void* stream)
{
	return b200_mamba2_mixer_prefill_host_ex(dtype, cfg, w, u_host, out_host, batch, seqlen, workspace, workspace_bytes, stream, 0);
}

// ---- head-sharded tensor parallelism ---------------------------------------------------------------------------------
namespace b200 {
int gated_mul_sumsq(int dtype, const void* x, int64_t xs, const void* z, int64_t zs, const void* w, void* y, int64_t ys,
	float* sumsq, int64_t rows, int64_t d, cudaStream_t st);
int row_scale_rsqrt(int dtype, void* out, int64_t ld, const float* sumsq, int64_t rows, int64_t cols, float inv_d, float eps,
	cudaStream_t st);

struct TpWs
{
	char* zxbcdt;
	char* xbc;
	char* y;
	char* ssd;
	size_t ssd_bytes, bytes;
	int64_t ldz;  // row stride of the local in_proj output: d_in_proj rounded up to 8 elements
};
static TpWs carve_tp(void* base, const b200_mamba2_config* c, const MixerDims& m, int64_t batch, int64_t seqlen)
{
	TpWs w;
	const size_t T = static_cast<size_t>(batch) * seqlen;
	w.ldz = (m.d_in_proj + 7) / 8 * 8;
	char* p = static_cast<char*>(base);
	size_t off = 0;
	w.zxbcdt = p + off; off += align_up(T * w.ldz * m.esz, 256);
	w.xbc = p + off; off += align_up(T * m.conv_dim * m.esz, 256);
	w.y = p + off; off += align_up(T * c->d_inner * m.esz, 256);
	w.ssd = p + off;
	w.ssd_bytes = b200_mamba_chunk_scan_combined_workspace_bytes(batch, seqlen, c->nheads, c->headdim, c->ngroups, c->d_state, c->chunk);
	off += w.ssd_bytes;
	w.bytes = off;
	return w;
}
}  // namespace b200

extern "C" size_t b200_mamba2_mixer_prefill_tp_workspace_bytes(const b200_mamba2_config* cfg_local, int dtype, int64_t batch,
	int64_t seqlen)
{
	MixerDims m;
	if (!dims_ok(cfg_local, dtype, &m) || batch <= 0 || seqlen <= 0) return 0;
	return carve_tp(nullptr, cfg_local, m, batch, seqlen).bytes;
}

extern "C" int b200_mamba2_mixer_prefill_tp_partial(int dtype, const b200_mamba2_config* cfg_local, const b200_mamba2_weights* w,
	const void* u, void* partial_out, float* sumsq, int64_t batch, int64_t seqlen, void* conv_state_out, float* ssm_state_out,
	void* workspace, size_t workspace_bytes, void* stream)
{
	if (!cfg_local || !w || !u || !partial_out || !sumsq) return B200_ERR_NULL;
	if (!w->in_proj_weight || !w->conv1d_weight || !w->conv1d_bias || !w->dt_bias || !w->A_log || !w->D || !w->norm_weight ||
		!w->out_proj_weight)
		return B200_ERR_NULL;
	MixerDims m;
	if (!dims_ok(cfg_local, dtype, &m) || batch < 0 || seqlen < 0) return B200_ERR_BAD_SHAPE;
	if (cfg_local->norm_group_size != 0 && cfg_local->norm_group_size != cfg_local->d_inner) return B200_ERR_UNSUPPORTED;
	if (batch == 0 || seqlen == 0) return B200_OK;
	if (!workspace) return B200_ERR_WORKSPACE;
	if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return B200_ERR_MISALIGNED;
	const TpWs ws = carve_tp(workspace, cfg_local, m, batch, seqlen);
	if (workspace_bytes < ws.bytes) return B200_ERR_WORKSPACE;
	const int64_t T = batch * seqlen;
	const int64_t d_inner = cfg_local->d_inner, GN = cfg_local->ngroups * cfg_local->d_state;
	const size_t e = m.esz;
	int rc = b200_linear(dtype, u, cfg_local->d_model, w->in_proj_weight, w->in_proj_layout, ws.zxbcdt, ws.ldz, T, cfg_local->d_model,
		ws.ldz, stream);
	if (rc) return rc;
	rc = b200_causal_conv1d_tokens(dtype, ws.zxbcdt + d_inner * e, ws.ldz, w->conv1d_weight, w->conv1d_bias, ws.xbc, m.conv_dim, nullptr,
		conv_state_out, batch, seqlen, m.conv_dim, static_cast<int>(cfg_local->d_conv), stream);
	if (rc) return rc;
	rc = b200_mamba_chunk_scan_combined(dtype, ws.xbc, m.conv_dim, ws.zxbcdt + (d_inner + m.conv_dim) * e, ws.ldz, w->A_log, 1,
		ws.xbc + d_inner * e, m.conv_dim, ws.xbc + (d_inner + GN) * e, m.conv_dim, w->D, w->dt_bias, nullptr, ws.y, d_inner,
		ssm_state_out, batch, seqlen, cfg_local->nheads, cfg_local->headdim, cfg_local->ngroups, cfg_local->d_state, cfg_local->chunk, B200_DT_SOFTPLUS_EXACT,
		ws.ssd, ws.ssd_bytes, stream);
	if (rc) return rc;
	rc = gated_mul_sumsq(dtype, ws.y, d_inner, ws.zxbcdt, ws.ldz, w->norm_weight, ws.y, d_inner, sumsq, T, d_inner,
		static_cast<cudaStream_t>(stream));
	if (rc) return rc;
	return b200_linear(dtype, ws.y, d_inner, w->out_proj_weight, w->out_proj_layout, partial_out, cfg_local->d_model, T, d_inner,
		cfg_local->d_model, stream);
}

extern "C" int b200_mamba2_mixer_tp_finish(int dtype, void* out, const float* sumsq, int64_t rows, int64_t d_model,
	int64_t d_inner_global, float eps, void* stream)
{
	if (!out || !sumsq) return B200_ERR_NULL;
	if (rows < 0 || d_model <= 0 || d_inner_global <= 0) return B200_ERR_BAD_SHAPE;
	if (dtype != B200_F16 && dtype != B200_F32) return B200_ERR_UNSUPPORTED;
	if (rows == 0) return B200_OK;
	return row_scale_rsqrt(dtype, out, d_model, sumsq, rows, d_model, 1.0f / static_cast<float>(d_inner_global), eps,
		static_cast<cudaStream_t>(stream));
}

// Decode workspace: zx | xbc | y | fp32 partial tiles of the stream-K projections | per-(row, head, warp) sums of squares.
struct DecodeLayout
{
	size_t zx, xbc, y, part, sumsq, total;
};

static DecodeLayout decode_layout(const b200_mamba2_config* cfg, const MixerDims& m, int dtype, int64_t batch)
{
	DecodeLayout L;
	size_t off = 0;
	L.zx = off;
	off += align_up(batch * m.ldz * m.esz, 256);
	L.xbc = off;
	off += align_up(batch * m.conv_dim * m.esz, 256);
	L.y = off;
	off += align_up(batch * cfg->d_inner * m.esz, 256);
	size_t p_in = 0, p_out = 0;
	if (decode_linear_applies(dtype, batch, cfg->d_model, m.d_in_proj)) p_in = decode_linear_partial_bytes(batch, cfg->d_model, m.d_in_proj);
	if (decode_linear_applies(dtype, batch, cfg->d_inner, cfg->d_model)) p_out = decode_linear_partial_bytes(batch, cfg->d_inner, cfg->d_model);
	L.part = off;
	off += p_in > p_out ? p_in : p_out;
	L.sumsq = off;
	off += align_up(batch * cfg->nheads * ssm_update_gated_partials() * sizeof(float), 256);  // one per warp of the recurrence kernel's CTAs
	L.total = off;
	return L;
}

extern "C" size_t b200_mamba2_mixer_decode_workspace_bytes(const b200_mamba2_config* cfg, int dtype, int64_t batch)
{
	MixerDims m;
	if (!dims_ok(cfg, dtype, &m) || batch <= 0) return 0;
	return decode_layout(cfg, m, dtype, batch).total;
}

// One token per sequence. With f16 tensors and at most 128 sequences the step is five launches:
//   stream-K in_proj -> slice sum + rolling conv1d/SiLU -> recurrence + gate (+ sums of squares) -> stream-K out_proj ->
//   slice sum + RMSNorm row scale.
// Otherwise the operators run one by one (linear, conv update, recurrence, gated RMSNorm, linear).
static int mixer_decode_impl(int dtype, const b200_mamba2_config* cfg, const b200_mamba2_weights* w,
	const void* u_t, void* out_t, void* conv_state, float* ssm_state, int64_t batch,
	void* workspace, size_t workspace_bytes, void* stream, const void* residual, int64_t ldr)
{
	if (!cfg || !w || !u_t || !out_t || !conv_state || !ssm_state) return B200_ERR_NULL;
	if (!w->in_proj_weight || !w->conv1d_weight || !w->conv1d_bias || !w->dt_bias || !w->A_log || !w->D || !w->norm_weight ||
		!w->out_proj_weight)
		return B200_ERR_NULL;
	MixerDims m;
	if (!dims_ok(cfg, dtype, &m) || batch < 0) return B200_ERR_BAD_SHAPE;
	if (batch == 0) return B200_OK;
	if (!workspace) return B200_ERR_WORKSPACE;
	if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return B200_ERR_MISALIGNED;
	const DecodeLayout L = decode_layout(cfg, m, dtype, batch);
	if (workspace_bytes < L.total) return B200_ERR_WORKSPACE;
	const size_t e = m.esz;
	char* base = static_cast<char*>(workspace);
	char* zx = base + L.zx;
	char* xbc = base + L.xbc;
	char* y = base + L.y;
	float* part = reinterpret_cast<float*>(base + L.part);
	float* sumsq = reinterpret_cast<float*>(base + L.sumsq);
	const int64_t d_inner = cfg->d_inner, GN = cfg->ngroups * cfg->d_state;
	cudaStream_t st = static_cast<cudaStream_t>(stream);
	const bool fuse_in = decode_linear_applies(dtype, batch, cfg->d_model, m.d_in_proj) && d_inner % 8 == 0 && m.conv_dim % 8 == 0;
	const bool fuse_out = decode_linear_applies(dtype, batch, d_inner, cfg->d_model);
	const bool whole_row_norm = cfg->norm_group_size == 0 || cfg->norm_group_size == d_inner;
	const bool fuse_gate = fuse_out && whole_row_norm && ssm_update_gated_applies(cfg->nheads, cfg->headdim, cfg->d_state, cfg->ngroups) && GN % 8 == 0;

	int rc;
	if (fuse_in)
	{
		rc = decode_in_proj_conv(u_t, cfg->d_model, w->in_proj_weight, w->in_proj_layout, zx, m.ldz, batch, cfg->d_model, m.d_in_proj,
			d_inner, m.conv_dim, static_cast<int>(cfg->d_conv), conv_state, w->conv1d_weight, w->conv1d_bias, xbc, part, st);
		if (rc) return rc;
	}
	else
	{
		rc = b200_linear(dtype, u_t, cfg->d_model, w->in_proj_weight, w->in_proj_layout, zx, m.ldz, batch, cfg->d_model,
			m.d_in_proj, stream);
		if (rc) return rc;
		rc = b200_causal_conv1d_update(dtype, zx + d_inner * e, m.ldz, conv_state, w->conv1d_weight, w->conv1d_bias, xbc,
			m.conv_dim, batch, m.conv_dim, static_cast<int>(cfg->d_conv), stream);
		if (rc) return rc;
	}
	if (fuse_gate)
	{
		rc = ssm_update_gated_f16(ssm_state, xbc, m.conv_dim, zx + (d_inner + m.conv_dim) * e, m.ldz, w->A_log, 1, xbc + d_inner * e,
			m.conv_dim, xbc + (d_inner + GN) * e, m.conv_dim, w->D, w->dt_bias, y, d_inner, zx, m.ldz, w->norm_weight, sumsq, batch,
			cfg->nheads, cfg->headdim, cfg->ngroups, cfg->d_state, 1, st);
		if (rc) return rc;
		return decode_out_proj_scale(y, d_inner, w->out_proj_weight, w->out_proj_layout, out_t, cfg->d_model, batch, d_inner, cfg->d_model,
			sumsq, static_cast<int>(cfg->nheads) * ssm_update_gated_partials(), d_inner, cfg->eps, part, st, residual, ldr);
	}
	rc = b200_selective_state_update(dtype, ssm_state, xbc, m.conv_dim, zx + (d_inner + m.conv_dim) * e, m.ldz, w->A_log, 1,
		xbc + d_inner * e, m.conv_dim, xbc + (d_inner + GN) * e, m.conv_dim, w->D, w->dt_bias, y, d_inner, batch, cfg->nheads,
		cfg->headdim, cfg->ngroups, cfg->d_state, 1, stream);
	if (rc) return rc;
	rc = b200_gated_rmsnorm(dtype, y, d_inner, zx, m.ldz, w->norm_weight, y, d_inner, batch, d_inner, cfg->norm_group_size,
		cfg->eps, stream);
	if (rc) return rc;
	if (fuse_out)
		return decode_out_proj_scale(y, d_inner, w->out_proj_weight, w->out_proj_layout, out_t, cfg->d_model, batch, d_inner, cfg->d_model,
			nullptr, 0, d_inner, cfg->eps, part, st, residual, ldr);
	return out_proj_residual(dtype, y, d_inner, w->out_proj_weight, w->out_proj_layout, out_t, cfg->d_model, batch, d_inner, cfg->d_model,
		residual, ldr, st);
}

extern "C" int b200_mamba2_mixer_decode(int dtype, const b200_mamba2_config* cfg, const b200_mamba2_weights* w,
	const void* u_t, void* out_t, void* conv_state, float* ssm_state, int64_t batch,
	void* workspace, size_t workspace_bytes, void* stream)
{
	return mixer_decode_impl(dtype, cfg, w, u_t, out_t, conv_state, ssm_state, batch, workspace, workspace_bytes, stream, nullptr, 0);
}

// ---- prefill continuation: `seqlen` more tokens of sequences whose state so far is in the cache ---------------------------
// Workspace: the next conv_state [b, conv_dim, d_conv-1] (written by the thread blocks that see the last tokens while others
// still read the old one, so it cannot be produced in place), then the prefill workspace.
extern "C" size_t b200_mamba2_mixer_prefill_continue_workspace_bytes(const b200_mamba2_config* cfg, int dtype, int64_t batch,
	int64_t seqlen)
{
	MixerDims m;
	if (!dims_ok(cfg, dtype, &m) || batch <= 0 || seqlen <= 0) return 0;
	return align_up(static_cast<size_t>(batch) * m.conv_dim * (cfg->d_conv - 1) * m.esz, 256) + carve_prefill(nullptr, cfg, m, batch, seqlen).bytes;
}

extern "C" int b200_mamba2_mixer_prefill_continue(int dtype, const b200_mamba2_config* cfg, const b200_mamba2_weights* w,
	const void* u, void* out, int64_t batch, int64_t seqlen, void* conv_state, float* ssm_state,
	void* workspace, size_t workspace_bytes, void* stream)
{
	if (!cfg || !w || !u || !out || !conv_state || !ssm_state) return B200_ERR_NULL;
	MixerDims m;
	if (!dims_ok(cfg, dtype, &m) || batch < 0 || seqlen < 0) return B200_ERR_BAD_SHAPE;
	if (batch == 0 || seqlen == 0) return B200_OK;
	if (!workspace) return B200_ERR_WORKSPACE;
	if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return B200_ERR_MISALIGNED;
	const size_t cs_bytes = static_cast<size_t>(batch) * m.conv_dim * (cfg->d_conv - 1) * m.esz;
	const size_t cs_pad = align_up(cs_bytes, 256);
	if (workspace_bytes < cs_pad + carve_prefill(nullptr, cfg, m, batch, seqlen).bytes) return B200_ERR_WORKSPACE;
	char* next_cs = static_cast<char*>(workspace);
	const int rc = mixer_prefill_impl(dtype, cfg, w, u, out, batch, seqlen, ssm_state, next_cs, ssm_state, next_cs + cs_pad,
		workspace_bytes - cs_pad, stream, nullptr, 0, conv_state);
	if (rc) return rc;
	if (cs_bytes) B200_CUDA_TRY(cudaMemcpyAsync(conv_state, next_cs, cs_bytes, cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(stream)));
	return B200_OK;
}

// ---- packed variable-length batches ------------------------------------------------------------------------------------------
// `nseq` sequences of different lengths stored back to back on the token axis: rows cu_seqlens[s] .. cu_seqlens[s+1]-1 of
// u / out belong to sequence s (cu_seqlens is a HOST array of nseq+1 non-decreasing offsets starting at 0, the convention of
// the `cu_seqlens` argument that scripts/zamba2/mamba_chunk_scan_comb.py:164-166 leaves unsupported). Both projections and the
// gated norm run once over all tokens; the conv1d and the scan, the two stages that look across tokens, run per sequence on
// its rows, so no padding is computed and nothing leaks across a boundary. An empty sequence leaves its initial state (or
// zeros) as its final state.
extern "C" size_t b200_mamba2_mixer_prefill_varlen_workspace_bytes(const b200_mamba2_config* cfg, int dtype, int64_t total_tokens)
{
	MixerDims m;
	if (!dims_ok(cfg, dtype, &m) || total_tokens <= 0) return 0;
	return carve_prefill(nullptr, cfg, m, 1, total_tokens).bytes;
}

extern "C" int b200_mamba2_mixer_prefill_varlen(int dtype, const b200_mamba2_config* cfg, const b200_mamba2_weights* w,
	const void* u, void* out, const int64_t* cu_seqlens, int64_t nseq,
	const float* initial_states, void* conv_state_out, float* ssm_state_out,
	void* workspace, size_t workspace_bytes, void* stream)
{
	if (!cfg || !w || !cu_seqlens) return B200_ERR_NULL;
	if (!w->in_proj_weight || !w->conv1d_weight || !w->conv1d_bias || !w->dt_bias || !w->A_log || !w->D || !w->norm_weight ||
		!w->out_proj_weight)
		return B200_ERR_NULL;
	MixerDims m;
	if (!dims_ok(cfg, dtype, &m) || nseq < 0 || cu_seqlens[0] != 0) return B200_ERR_BAD_SHAPE;
	for (int64_t s = 0; s < nseq; ++s)
		if (cu_seqlens[s + 1] < cu_seqlens[s]) return B200_ERR_BAD_SHAPE;
	const int64_t T = cu_seqlens[nseq];
	cudaStream_t st = static_cast<cudaStream_t>(stream);
	const size_t e = m.esz;
	const int64_t d_inner = cfg->d_inner;
	const size_t state_elems = static_cast<size_t>(cfg->nheads) * cfg->headdim * cfg->d_state;
	const size_t cs_bytes = static_cast<size_t>(m.conv_dim) * (cfg->d_conv - 1) * e;
	PrefillWs ws{};
	if (T > 0)
	{
		if (!u || !out) return B200_ERR_NULL;
		if (!workspace) return B200_ERR_WORKSPACE;
		if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return B200_ERR_MISALIGNED;
		ws = carve_prefill(workspace, cfg, m, 1, T);
		if (workspace_bytes < ws.bytes) return B200_ERR_WORKSPACE;
		const int rc = b200_linear(dtype, u, cfg->d_model, w->in_proj_weight, w->in_proj_layout, ws.zxbcdt, m.ldz, T, cfg->d_model,
			m.d_in_proj, stream);
		if (rc) return rc;
	}
	// f16 with the shapes of the one-kernel scan: conv1d + dt stage of all sequences in one launch, the scan in another. Taken
	// unless the index arrays and the per-block dt rows do not fit the scan's scratch area (very many empty sequences).
	bool packed_done = false;
	if (T > 0 && mixer_varlen_fused_applies(dtype, ws.zxbcdt + d_inner * e, m.ldz, ws.xbc, m.conv_dim, w->conv1d_weight, w->conv1d_bias,
			static_cast<int>(cfg->d_conv), T, nseq, cfg->nheads, cfg->headdim, cfg->ngroups, cfg->d_state, ws.y, d_inner, initial_states,
			ssm_state_out))
	{
		const int rc = mixer_conv_ssd_varlen_f16(ws.zxbcdt + d_inner * e, m.ldz, w->conv1d_weight, w->conv1d_bias, static_cast<int>(cfg->d_conv),
			ws.xbc, m.conv_dim, conv_state_out, ws.zxbcdt + (d_inner + m.conv_dim) * e, m.ldz, w->A_log, w->dt_bias, w->D, initial_states, ws.y,
			d_inner, ssm_state_out, cu_seqlens, nseq, cfg->nheads, cfg->headdim, cfg->ngroups, cfg->d_state, ws.ssd, ws.ssd_bytes, st);
		if (rc == B200_OK)
		{
			packed_done = true;
			// an empty sequence: its final state is its initial state (the scan kernel copies it), its conv_state is zero
			for (int64_t s = 0; s < nseq && conv_state_out && cs_bytes; ++s)
				if (cu_seqlens[s + 1] == cu_seqlens[s])
					B200_CUDA_TRY(cudaMemsetAsync(static_cast<char*>(conv_state_out) + s * cs_bytes, 0, cs_bytes, st));
		}
		else if (rc != B200_ERR_WORKSPACE)
			return rc;
	}
	for (int64_t s = 0; s < nseq && !packed_done; ++s)
	{
		const int64_t t0 = cu_seqlens[s], len = cu_seqlens[s + 1] - t0;
		const float* init = initial_states ? initial_states + s * state_elems : nullptr;
		float* fin = ssm_state_out ? ssm_state_out + s * state_elems : nullptr;
		char* cs = conv_state_out ? static_cast<char*>(conv_state_out) + s * cs_bytes : nullptr;
		if (len == 0)
		{
			if (fin && init && fin != init)
				B200_CUDA_TRY(cudaMemcpyAsync(fin, init, state_elems * sizeof(float), cudaMemcpyDeviceToDevice, st));
			else if (fin && !init)
				B200_CUDA_TRY(cudaMemsetAsync(fin, 0, state_elems * sizeof(float), st));
			if (cs && cs_bytes) B200_CUDA_TRY(cudaMemsetAsync(cs, 0, cs_bytes, st));
			continue;
		}
		const int rc = mixer_conv_ssd(dtype, cfg, w, m, ws.zxbcdt + t0 * m.ldz * e, ws.xbc + t0 * m.conv_dim * e,
			ws.y + t0 * d_inner * e, ws.ssd, ws.ssd_bytes, 1, len, init, nullptr, cs, fin, st, false);
		if (rc) return rc;
	}
	if (T == 0) return B200_OK;
	int rc = b200_gated_rmsnorm(dtype, ws.y, d_inner, ws.zxbcdt, m.ldz, w->norm_weight, ws.y, d_inner, T, d_inner,
		cfg->norm_group_size, cfg->eps, stream);
	if (rc) return rc;
	return b200_linear(dtype, ws.y, d_inner, w->out_proj_weight, w->out_proj_layout, out, cfg->d_model, T, d_inner, cfg->d_model, stream);
}

// ---- sequence-parallel prefill: one sequence split into segments, one segment per GPU ----------------------------------------
// Everything but the scan's state is local to a segment once the d_conv-1 tokens before it are known (they are re-projected
// here: cheaper than shipping conv inputs). The state is linear in what enters the segment: begin() runs in_proj, conv1d and the
// per-chunk states and reports the segment's outgoing state for a ZERO incoming state plus the log of its total decay;
// after the ranks have exchanged those two small tensors, b200_ssm_segment_prefix folds them into the true incoming state
// and finish() runs the state passing, the chunk scan, the gated norm and out_proj. The library does not communicate.
// Workspace: projected halo [b*(d_conv-1), d_in_proj] | halo conv_state [b, conv_dim, d_conv-1] | halo conv output (unused) | the prefill workspace, which
// must be handed unchanged from begin() to finish().
namespace b200 {
struct SpWs
{
	char* halo_zx;
	char* halo_cs;
	char* halo_y;
	char* inner;
	size_t inner_bytes, bytes;
};
static SpWs carve_sp(void* base, const b200_mamba2_config* c, const MixerDims& m, int64_t batch, int64_t seglen)
{
	SpWs w;
	char* p = static_cast<char*>(base);
	size_t off = 0;
	const int64_t hw = c->d_conv - 1;
	w.halo_zx = p + off; off += align_up(static_cast<size_t>(batch) * hw * m.ldz * m.esz, 256);
	w.halo_cs = p + off; off += align_up(static_cast<size_t>(batch) * m.conv_dim * hw * m.esz, 256);
	w.halo_y = p + off; off += align_up(static_cast<size_t>(batch) * m.conv_dim * hw * m.esz, 256);
	w.inner = p + off;
	w.inner_bytes = carve_prefill(nullptr, c, m, batch, seglen).bytes;
	w.bytes = off + w.inner_bytes;
	return w;
}
}  // namespace b200

extern "C" size_t b200_mamba2_mixer_prefill_sp_workspace_bytes(const b200_mamba2_config* cfg, int dtype, int64_t batch, int64_t seglen)
{
	MixerDims m;
	if (!dims_ok(cfg, dtype, &m) || batch <= 0 || seglen <= 0) return 0;
	return carve_sp(nullptr, cfg, m, batch, seglen).bytes;
}

extern "C" int b200_mamba2_mixer_prefill_sp_begin(int dtype, const b200_mamba2_config* cfg, const b200_mamba2_weights* w,
	const void* u_seg, const void* u_halo, int64_t batch, int64_t seglen, float* seg_state, float* seg_logdecay, void* conv_state_out,
	void* workspace, size_t workspace_bytes, void* stream)
{
	if (!cfg || !w || !u_seg || !seg_state || !seg_logdecay) return B200_ERR_NULL;
	if (!w->in_proj_weight || !w->conv1d_weight || !w->conv1d_bias || !w->dt_bias || !w->A_log) return B200_ERR_NULL;
	MixerDims m;
	if (!dims_ok(cfg, dtype, &m) || batch <= 0 || seglen <= 0) return B200_ERR_BAD_SHAPE;
	if (!workspace) return B200_ERR_WORKSPACE;
	if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return B200_ERR_MISALIGNED;
	const SpWs sp = carve_sp(workspace, cfg, m, batch, seglen);
	if (workspace_bytes < sp.bytes) return B200_ERR_WORKSPACE;
	const PrefillWs ws = carve_prefill(sp.inner, cfg, m, batch, seglen);
	const int64_t T = batch * seglen, d_inner = cfg->d_inner, GN = cfg->ngroups * cfg->d_state, hw = cfg->d_conv - 1;
	const size_t e = m.esz;
	cudaStream_t st = static_cast<cudaStream_t>(stream);
	int rc;
	const void* conv_in = nullptr;
	if (u_halo != nullptr && hw > 0)
	{
		// the conv inputs of the d_conv-1 tokens before the segment: project them and let the conv kernel lay them out as a state
		rc = b200_linear(dtype, u_halo, cfg->d_model, w->in_proj_weight, w->in_proj_layout, sp.halo_zx, m.ldz, batch * hw, cfg->d_model,
			m.d_in_proj, stream);
		if (rc) return rc;
		rc = b200_causal_conv1d_tokens(dtype, sp.halo_zx + d_inner * e, m.ldz, w->conv1d_weight, w->conv1d_bias, sp.halo_y /* unused */,
			m.conv_dim, nullptr, sp.halo_cs, batch, hw, m.conv_dim, static_cast<int>(cfg->d_conv), stream);
		if (rc) return rc;
		conv_in = sp.halo_cs;
	}
	rc = b200_linear(dtype, u_seg, cfg->d_model, w->in_proj_weight, w->in_proj_layout, ws.zxbcdt, m.ldz, T, cfg->d_model, m.d_in_proj,
		stream);
	if (rc) return rc;
	const char* dtp = ws.zxbcdt + (d_inner + m.conv_dim) * e;
	rc = b200_causal_conv1d_tokens(dtype, ws.zxbcdt + d_inner * e, m.ldz, w->conv1d_weight, w->conv1d_bias, ws.xbc, m.conv_dim, conv_in,
		conv_state_out, batch, seglen, m.conv_dim, static_cast<int>(cfg->d_conv), stream);
	if (rc) return rc;
	rc = ssd_combined_stages(dtype, ws.xbc, m.conv_dim, dtp, m.ldz, w->A_log, 1, ws.xbc + d_inner * e, m.conv_dim,
		ws.xbc + (d_inner + GN) * e, m.conv_dim, w->D, w->dt_bias, nullptr, ws.y, d_inner, seg_state, batch, seglen, cfg->nheads, cfg->headdim,
		cfg->ngroups, cfg->d_state, cfg->chunk, B200_DT_SOFTPLUS_EXACT, ws.ssd, ws.ssd_bytes, stream,
		kSsdStageDt | kSsdStageStates | kSsdStageSummary);
	if (rc) return rc;
	return ssd_segment_logdecay_of(seg_logdecay, batch, seglen, cfg->nheads, cfg->headdim, cfg->ngroups, cfg->d_state, cfg->chunk, ws.ssd, st);
}

extern "C" int b200_ssm_segment_prefix(const float* seg_states, const float* seg_logdecay, int nseg, int64_t batch, int64_t H, int64_t P,
	int64_t N, float* state_in, void* stream)
{
	if (!state_in || (nseg > 0 && (!seg_states || !seg_logdecay))) return B200_ERR_NULL;
	if (nseg < 0 || batch < 0 || H <= 0 || P <= 0 || N <= 0) return B200_ERR_BAD_SHAPE;
	if (batch == 0) return B200_OK;
	return ssd_segment_prefix(seg_states, seg_logdecay, nseg, batch, H, P, N, state_in, static_cast<cudaStream_t>(stream));
}

extern "C" int b200_mamba2_mixer_prefill_sp_finish(int dtype, const b200_mamba2_config* cfg, const b200_mamba2_weights* w, void* out_seg,
	int64_t batch, int64_t seglen, const float* state_in, float* ssm_state_out, void* workspace, size_t workspace_bytes, void* stream)
{
	if (!cfg || !w || !out_seg) return B200_ERR_NULL;
	if (!w->A_log || !w->D || !w->dt_bias || !w->norm_weight || !w->out_proj_weight) return B200_ERR_NULL;
	MixerDims m;
	if (!dims_ok(cfg, dtype, &m) || batch <= 0 || seglen <= 0) return B200_ERR_BAD_SHAPE;
	if (!workspace) return B200_ERR_WORKSPACE;
	if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return B200_ERR_MISALIGNED;
	const SpWs sp = carve_sp(workspace, cfg, m, batch, seglen);
	if (workspace_bytes < sp.bytes) return B200_ERR_WORKSPACE;
	const PrefillWs ws = carve_prefill(sp.inner, cfg, m, batch, seglen);
	const int64_t T = batch * seglen, d_inner = cfg->d_inner, GN = cfg->ngroups * cfg->d_state;
	const size_t e = m.esz;
	const char* dtp = ws.zxbcdt + (d_inner + m.conv_dim) * e;
	int rc = ssd_combined_stages(dtype, ws.xbc, m.conv_dim, dtp, m.ldz, w->A_log, 1, ws.xbc + d_inner * e, m.conv_dim,
		ws.xbc + (d_inner + GN) * e, m.conv_dim, w->D, w->dt_bias, state_in, ws.y, d_inner, ssm_state_out, batch, seglen, cfg->nheads,
		cfg->headdim, cfg->ngroups, cfg->d_state, cfg->chunk, B200_DT_SOFTPLUS_EXACT, ws.ssd, ws.ssd_bytes, stream, kSsdStagePass);
	if (rc) return rc;
	rc = b200_gated_rmsnorm(dtype, ws.y, d_inner, ws.zxbcdt, m.ldz, w->norm_weight, ws.y, d_inner, T, d_inner, cfg->norm_group_size,
		cfg->eps, stream);
	if (rc) return rc;
	return b200_linear(dtype, ws.y, d_inner, w->out_proj_weight, w->out_proj_layout, out_seg, cfg->d_model, T, d_inner, cfg->d_model, stream);
}

// ---- Zamba2 Mamba decoder layer around the mixer: out = hidden + mixer(rms_norm(hidden) * input_norm_weight) -------------
// Workspace: the normalised hidden states [T, d_model], then the mixer's own workspace.
extern "C" size_t b200_mamba2_decoder_prefill_workspace_bytes(const b200_mamba2_config* cfg, int dtype, int64_t batch, int64_t seqlen)
{
	const size_t inner = b200_mamba2_mixer_prefill_workspace_bytes(cfg, dtype, batch, seqlen);
	if (inner == 0) return 0;
	return align_up(static_cast<size_t>(batch) * seqlen * cfg->d_model * (dtype == B200_F16 ? 2 : 4), 256) + inner;
}

extern "C" int b200_mamba2_decoder_prefill(int dtype, const b200_mamba2_config* cfg, const b200_mamba2_weights* w,
	const void* input_norm_weight, float rms_eps, const void* hidden, void* out, int64_t batch, int64_t seqlen,
	const float* initial_states, void* conv_state_out, float* ssm_state_out, void* workspace, size_t workspace_bytes, void* stream)
{
	if (!cfg || !w || !input_norm_weight || !hidden || !out) return B200_ERR_NULL;
	if (dtype != B200_F16 && dtype != B200_F32) return B200_ERR_UNSUPPORTED;
	if (batch < 0 || seqlen < 0 || cfg->d_model <= 0) return B200_ERR_BAD_SHAPE;
	if (batch == 0 || seqlen == 0) return B200_OK;
	if (!workspace) return B200_ERR_WORKSPACE;
	if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return B200_ERR_MISALIGNED;
	const size_t need = b200_mamba2_decoder_prefill_workspace_bytes(cfg, dtype, batch, seqlen);
	if (need == 0) return B200_ERR_BAD_SHAPE;
	if (workspace_bytes < need) return B200_ERR_WORKSPACE;
	const int64_t T = batch * seqlen;
	const size_t normed_bytes = align_up(static_cast<size_t>(T) * cfg->d_model * (dtype == B200_F16 ? 2 : 4), 256);
	char* normed = static_cast<char*>(workspace);
	int rc = b200_rms_norm(dtype, hidden, cfg->d_model, input_norm_weight, normed, cfg->d_model, T, cfg->d_model, rms_eps, 0, stream);
	if (rc) return rc;
	return mixer_prefill_impl(dtype, cfg, w, normed, out, batch, seqlen, initial_states, conv_state_out, ssm_state_out,
		normed + normed_bytes, workspace_bytes - normed_bytes, stream, hidden, cfg->d_model);
}

extern "C" size_t b200_mamba2_decoder_decode_workspace_bytes(const b200_mamba2_config* cfg, int dtype, int64_t batch)
{
	const size_t inner = b200_mamba2_mixer_decode_workspace_bytes(cfg, dtype, batch);
	if (inner == 0) return 0;
	return align_up(static_cast<size_t>(batch) * cfg->d_model * (dtype == B200_F16 ? 2 : 4), 256) + inner;
}

extern "C" int b200_mamba2_decoder_decode(int dtype, const b200_mamba2_config* cfg, const b200_mamba2_weights* w,
	const void* input_norm_weight, float rms_eps, const void* hidden_t, void* out_t, void* conv_state, float* ssm_state, int64_t batch,
	void* workspace, size_t workspace_bytes, void* stream)
{
	if (!cfg || !w || !input_norm_weight || !hidden_t || !out_t) return B200_ERR_NULL;
	if (dtype != B200_F16 && dtype != B200_F32) return B200_ERR_UNSUPPORTED;
	if (batch < 0 || cfg->d_model <= 0) return B200_ERR_BAD_SHAPE;
	if (batch == 0) return B200_OK;
	if (!workspace) return B200_ERR_WORKSPACE;
	if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return B200_ERR_MISALIGNED;
	const size_t need = b200_mamba2_decoder_decode_workspace_bytes(cfg, dtype, batch);
	if (need == 0) return B200_ERR_BAD_SHAPE;
	if (workspace_bytes < need) return B200_ERR_WORKSPACE;
	const size_t normed_bytes = align_up(static_cast<size_t>(batch) * cfg->d_model * (dtype == B200_F16 ? 2 : 4), 256);
	char* normed = static_cast<char*>(workspace);
	int rc = b200_rms_norm(dtype, hidden_t, cfg->d_model, input_norm_weight, normed, cfg->d_model, batch, cfg->d_model, rms_eps, 0, stream);
	if (rc) return rc;
	return mixer_decode_impl(dtype, cfg, w, normed, out_t, conv_state, ssm_state, batch, normed + normed_bytes,
		workspace_bytes - normed_bytes, stream, hidden_t, cfg->d_model);
}
