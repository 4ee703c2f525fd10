/*
 * b200_mamba2.h - C ABI of the B200 (sm_100a) Mamba2-mixer forward path.
 *
 * This is the boundary a host program binds against when it replaces anyGPU's operators for the
 * Mamba2 mixer of its Zamba2 blocks. anyGPU has no FFI: its boundary is the set of C++ host launchers
 * `cu_<op>_<dtype>(const Tensor<..,CUDA>&, ..., Tensor<..,CUDA>& out)` declared in srcs/kernels/cuda/*.cuh
 * and called by the `tensor_<op>` templates in srcs/ops, srcs/fused and srcs/models/zamba2. Each entry
 * point below names the launcher / template it stands in for. The C++ header layer under
 * include/anygpu/ re-creates the `tensor_<op>` templates on top of this ABI.
 *
 * Conventions
 *  - every pointer is a DEVICE pointer unless its name ends in `_host`;
 *  - tensors are row-major; `*_stride` arguments are element strides between consecutive rows (tokens)
 *    so that slices of a wider buffer (z | xBC | dt inside the in_proj output) are consumed in place;
 *  - `dtype` selects the storage type of activations and weights (B200_F16 or B200_F32); the scan
 *    parameters A / A_log, D, dt_bias, the SSM state and all statistics are always fp32;
 *  - `stream` is a cudaStream_t passed as void*; all work is stream-ordered and nothing synchronises;
 *  - no entry point allocates device memory: scratch comes from the caller's `workspace`
 *    (size from the matching *_workspace_bytes query), 256-byte aligned;
 *  - the return value is 0 on success or a negative b200_status; nothing calls exit().
 *  - f16 rows must start on 16-byte boundaries (row strides multiples of 8 elements) for the vectorised
 *    kernels; shapes that break this take a scalar kernel where one exists or return B200_ERR_MISALIGNED.
 */
#ifndef B200_MAMBA2_H
#define B200_MAMBA2_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#pragma GCC visibility push(default)
#endif
#ifdef __cplusplus
extern "C" {
#endif

typedef enum b200_status
{
	B200_OK = 0,
	B200_ERR_BAD_SHAPE = -1,      /* a dimension is zero/negative or inconsistent with another */
	B200_ERR_MISALIGNED = -2,     /* pointer or stride alignment required by the kernel is not met */
	B200_ERR_WORKSPACE = -3,      /* workspace null or smaller than *_workspace_bytes reports */
	B200_ERR_DEVICE_TIMEOUT = -4, /* a bounded device-side wait gave up (reported by b200_last_device_error) */
	B200_ERR_CUDA = -5,           /* a CUDA runtime / driver call failed; see b200_last_cuda_error() */
	B200_ERR_UNSUPPORTED = -6,    /* dtype / size combination that no kernel covers */
	B200_ERR_NULL = -7            /* a required pointer is null */
} b200_status;

typedef enum b200_dtype
{
	B200_F16 = 0,
	B200_F32 = 1
} b200_dtype;

/* Layout of a projection weight handed to b200_linear. */
typedef enum b200_weight_layout
{
	B200_W_KN = 0, /* (in_features, out_features) row-major: what anyGPU's tensor_linear takes (srcs/ops/mm_ops.hpp:206-232) */
	B200_W_NK = 1  /* (out_features, in_features) row-major: the torch / checkpoint layout before anyGPU's load-time transpose
	                  (srcs/models/zamba2/zamba_mlp.hpp:26-29) */
} b200_weight_layout;

const char* b200_status_string(int status);
/* Last cudaError_t (as int) recorded by a failing call on this host thread, 0 if none. */
int b200_last_cuda_error(void);
/* ABI version; bumped when a signature changes. */
int b200_abi_version(void);
/* Number of kernel launches the library has issued in this process since the last call with reset != 0 (a benchmark harness
 * counts the launches of its timed region with it). No counterpart in anyGPU. */
long long b200_launch_count(int reset);
/* Reads (and clears) the device-side error word that bounded waits set. Synchronises `stream`.
 * Returns B200_OK or B200_ERR_DEVICE_TIMEOUT; *detail (optional) receives the raw word. */
int b200_last_device_error(void* stream, uint32_t* detail);

/* ---- Y[M,N] = X[M,K] . W ------------------------------------------------------------------------------
 * Replaces opt2::cu_tensor_mm_f16 (srcs/kernels/cuda/mm_ops.cu:231-350) and cu_tensor_mm_f32_opt0
 * (mm_ops.cu:7-51) behind tensor_mm / tensor_linear (srcs/ops/mm_ops.hpp:48-71,206-232).
 * f16: tcgen05 tensor-core kernels with fp32 accumulation when K, N, ldx, ldy are multiples of 8 and x, w, y start on 16-byte
 * boundaries (what TMA can address); any other f16 shape runs on a SIMT kernel (fp32 accumulation), as tensor_linear accepts
 * every shape. f32: exact fp32 SIMT kernel.  ldx / ldy: row strides of X and Y in elements. */
int b200_linear(int dtype, const void* x, int64_t ldx, const void* w, int w_layout, void* y, int64_t ldy,
	int64_t M, int64_t K, int64_t N, void* stream);
/* Name of the kernel b200_linear launches for a problem of this size (for aligned operands): what a profile of the call shows. */
const char* b200_linear_kernel_name(int dtype, int64_t M, int64_t K, int64_t N);

/* Self-test of the give-up path of the bounded device-side waits (no counterpart in anyGPU). Runs the single-CTA f16 kernel of
 * b200_linear on the given problem with its TMA producer told to leave out the last K-block of every tile, and with the poll
 * limit of the kernel's waits lowered to `spin_limit`: the MMA-issuing thread waits for a stage that never fills, gives up after
 * that many polls, the CTA records the site in the device error word, lets its copies and MMAs in flight land, frees its tensor
 * memory and returns - no trap, no fault, the context stays usable. Y holds no meaningful result afterwards. The call returns
 * B200_OK (the launch succeeded); b200_last_device_error then reports B200_ERR_DEVICE_TIMEOUT. f16 only; problems large enough
 * for the CTA-pair kernel are rejected with B200_ERR_UNSUPPORTED. */
int b200_debug_linear_starved_producer(const void* x, int64_t ldx, const void* w, int w_layout, void* y, int64_t ldy, int64_t M,
	int64_t K, int64_t N, uint32_t spin_limit, void* stream);

/* ---- causal conv1d + SiLU, (batch, dims, seq_len) layout ---------------------------------------------------
 * Replaces cu_tensor_causal_conv1d_f32 (srcs/kernels/cuda/causal_conv1d.cu:78-101) behind
 * tensor_causal_conv1d (srcs/fused/causal_conv1d.hpp:90-117). y[b,d,s] = silu(bias[d] + sum_k w[d,k] x[b,d,s+k-(W-1)]),
 * zero left padding, fp32 accumulation. width in [1,4]. w is (dims, width), bias (dims). */
int b200_causal_conv1d(int dtype, const void* x, const void* w, const void* bias, void* y,
	int64_t batch, int64_t dims, int64_t seqlen, int width, void* stream);

/* Same operator on token-major data: x is [batch, seqlen, dims] with row stride x_stride (so the xBC slice of
 * the in_proj output is read in place, without anyGPU's tensor_slice + tensor_transp round trip,
 * srcs/ops/shape_ops.hpp:190-254, srcs/ops/transp_ops.hpp:81-134). y likewise with y_stride.
 * initial_state (optional) is [batch, dims, width-1] holding the inputs that precede the sequence (oldest first);
 * final_state (optional) receives the last width-1 inputs in the same layout (the decode conv_state). */
int b200_causal_conv1d_tokens(int dtype, const void* x, int64_t x_stride, const void* w, const void* bias,
	void* y, int64_t y_stride, const void* initial_state, void* final_state,
	int64_t batch, int64_t seqlen, int64_t dims, int width, void* stream);

/* One decode step: conv_state [batch, dims, width-1] (oldest first) is read, the output for token x_t
 * [batch, dims] (row stride x_stride) is written to y_t (row stride y_stride), and the state is advanced in place.
 * No counterpart in anyGPU (its backlog lists the mamba layer as open, docs/TODO_backlog.md:3-25);
 * defined so that step t reproduces column t of tensor_causal_conv1d on the concatenated history. */
int b200_causal_conv1d_update(int dtype, const void* x_t, int64_t x_stride, void* conv_state, const void* w,
	const void* bias, void* y_t, int64_t y_stride, int64_t batch, int64_t dims, int width, void* stream);

/* ---- gated RMSNorm ------------------------------------------------------------------------------------------
 * Replaces the three launches of tensor_zamba_gated_rmsnorm (srcs/models/zamba2/zamba_gated_rmsnorm.hpp:9-23):
 * cu_tensor_silu_f32 (srcs/kernels/cuda/math_ops.cu:3-34), cu_tensor_mul_f32 (binary_ops.cu:112-124),
 * cu_tensor_rms_norm_f32_v1 (norm_rms_f32_v1.cu:94-119) by one pass:
 * g = x * silu(z); y = g * rsqrt(mean_group(g^2) + eps) * w.  group_size must divide d; group_size == d is
 * anyGPU's behaviour (it ignores its gsize argument). */
int b200_gated_rmsnorm(int dtype, const void* x, int64_t x_stride, const void* z, int64_t z_stride, const void* w,
	void* y, int64_t y_stride, int64_t rows, int64_t d, int64_t group_size, float eps, void* stream);

/* ---- RMSNorm over the last axis ----------------------------------------------------------------------------
 * tensor_rms_norm(x, -1, w, eps, zero_centered) (srcs/ops/norm_ops.hpp:134-228; CUDA launcher cu_tensor_rms_norm_f32_v1,
 * srcs/kernels/cuda/norm_rms_f32_v1.cu:94-119, f32 only there): y = x * rsqrt(mean_row(x^2) + eps) * (w + delta), delta = 1 when
 * zero_centered != 0. x [rows, dim] (row stride x_stride), w [dim], y [rows, dim] (row stride y_stride). */
int b200_rms_norm(int dtype, const void* x, int64_t x_stride, const void* w, void* y, int64_t y_stride, int64_t rows, int64_t dim,
	float eps, int zero_centered, void* stream);

/* ---- SSD chunked selective scan (prefill) -------------------------------------------------------------------
 * CUDA counterpart of mamba_chunk_scan_combined_ref (scripts/zamba2/mamba_chunk_scan_comb.py:167-215), which anyGPU
 * has only as a PyTorch script. Argument meaning follows that function:
 *   x [b,l,H,P] (token stride x_stride), dt [b,l,H] (dt_stride), A [H] fp32 (or A_log when a_is_log != 0: A = -exp(A_log)),
 *   B, C [b,l,G,N] (B_stride, C_stride), D [H] fp32 or null, dt_bias [H] fp32 or null,
 *   initial_states [b,H,P,N] fp32 or null  ->  y [b,l,H,P] (y_stride), final_states [b,H,P,N] fp32 (or null).
 * chunk <= 256. seqlen need not be a multiple of chunk: y is exact either way; final_states follows dt_softplus:
 *   B200_DT_SOFTPLUS (1)        the script's behaviour: it pads dt with zeros BEFORE bias and softplus (:38-45), so the padded
 *                               tail of the last chunk decays final_states by exp(A * softplus(dt_bias)) per padded position;
 *   B200_DT_SOFTPLUS_EXACT (2)  padded positions carry dt = 0: final_states is the state after the last real token (what a
 *                               decode step or a further prefill piece must start from). The mixer entry points use this. */
#define B200_DT_SOFTPLUS 1
#define B200_DT_SOFTPLUS_EXACT 2
size_t b200_mamba_chunk_scan_combined_workspace_bytes(int64_t batch, int64_t seqlen, int64_t H, int64_t P, int64_t G,
	int64_t N, int64_t chunk);
int b200_mamba_chunk_scan_combined(int dtype, const void* x, int64_t x_stride, const void* dt, int64_t dt_stride,
	const float* A, int a_is_log, const void* B, int64_t B_stride, const void* C, int64_t C_stride,
	const float* D, const float* dt_bias, const float* initial_states,
	void* y, int64_t y_stride, float* final_states,
	int64_t batch, int64_t seqlen, int64_t H, int64_t P, int64_t G, int64_t N, int64_t chunk, int dt_softplus,
	void* workspace, size_t workspace_bytes, void* stream);

/* Same operator for callers that cannot provide a workspace. No counterpart in anyGPU (it allocates every operator
 * output with cudaMalloc, srcs/core/tensor.hpp:80-84): this variant exists for hosts that may not allocate device memory at
 * all - a plugin that only receives its input and output tensors from a runtime owning the allocator, code inside a region
 * where cudaMalloc is not permitted, a binding whose pool is exhausted. The scratch is a fixed array inside the library's
 * device image: b200_mamba_chunk_scan_combined_static_capacity() bytes (64 MiB) are held on every GPU that loads the
 * library until the process exits. Problems whose workspace (b200_mamba_chunk_scan_combined_workspace_bytes) exceeds that
 * capacity are rejected with B200_ERR_WORKSPACE. The call itself allocates nothing. Its FIRST call on each device looks up
 * the array's device address (cudaGetSymbolAddress); make that first call outside any stream capture. All calls share the
 * one array and it keeps the previous call's contents (harmless: each stage overwrites what the next one reads), so two calls
 * whose kernels can overlap on the GPU - different streams, or different host threads - race on it: issue them on one stream. */
size_t b200_mamba_chunk_scan_combined_static_capacity(void);
int b200_mamba_chunk_scan_combined_static(int dtype, const void* x, int64_t x_stride, const void* dt, int64_t dt_stride,
	const float* A, int a_is_log, const void* B, int64_t B_stride, const void* C, int64_t C_stride,
	const float* D, const float* dt_bias, const float* initial_states,
	void* y, int64_t y_stride, float* final_states,
	int64_t batch, int64_t seqlen, int64_t H, int64_t P, int64_t G, int64_t N, int64_t chunk, int dt_softplus, void* stream);

/* ---- single-token state recurrence (decode) -----------------------------------------------------------------
 * dt = softplus(dt_raw + dt_bias); h <- exp(dt A) h + dt x (x) B; y = h.C + D x, per (batch, head).
 * ssm_state [b,H,P,N] fp32 is updated in place. No counterpart in anyGPU; equals one step of the per-token form of
 * mamba_chunk_scan_combined_ref with initial_states (scripts/zamba2/mamba_chunk_scan_comb.py:93-95,196-210).
 * x [b,H,P] (row stride x_stride), dt [b,H], B, C [b,G,N], y [b,H,P]. */
int b200_selective_state_update(int dtype, float* ssm_state, const void* x, int64_t x_stride, const void* dt, int64_t dt_stride,
	const float* A, int a_is_log, const void* B, int64_t B_stride, const void* C, int64_t C_stride,
	const float* D, const float* dt_bias, void* y, int64_t y_stride,
	int64_t batch, int64_t H, int64_t P, int64_t G, int64_t N, int dt_softplus, void* stream);

/* ---- the mixer ----------------------------------------------------------------------------------------------
 * The block anyGPU was building towards (docs/TODO_backlog.md:3-25), composed as
 *   zxbcdt = in_proj(u) ; z | xBC | dt ; xBC = silu(conv1d(xBC)) ; x | B | C ; y = SSD(...) ;
 *   g = gated_rmsnorm(y, z) ; out = out_proj(g)
 * in the style of its other Zamba2 blocks (weights struct + cache + config, srcs/models/zamba2/zamba_attn_decoder.hpp:68-118). */
typedef struct b200_mamba2_config
{
	int64_t d_model, d_inner, nheads, headdim, d_state, ngroups, d_conv, chunk;
	int64_t norm_group_size; /* 0 = whole row (anyGPU's gated RMSNorm behaviour) */
	float eps;
} b200_mamba2_config;

typedef struct b200_mamba2_weights
{
	const void* in_proj_weight;  /* dtype, layout in_proj_layout: [d_model, d_in_proj] (KN) or [d_in_proj, d_model] (NK) */
	const void* conv1d_weight;   /* dtype [conv_dim, d_conv] */
	const void* conv1d_bias;     /* dtype [conv_dim] */
	const float* dt_bias;        /* fp32 [nheads] */
	const float* A_log;          /* fp32 [nheads] */
	const float* D;              /* fp32 [nheads] */
	const void* norm_weight;     /* dtype [d_inner] */
	const void* out_proj_weight; /* dtype, layout out_proj_layout */
	int in_proj_layout, out_proj_layout; /* b200_weight_layout */
} b200_mamba2_weights;

size_t b200_mamba2_mixer_prefill_workspace_bytes(const b200_mamba2_config* cfg, int dtype, int64_t batch, int64_t seqlen);
/* u [batch, seqlen, d_model] -> out [batch, seqlen, d_model]. initial_states / ssm_state_out [b,H,P,N] fp32 and
 * conv_state_out [b, conv_dim, d_conv-1] (dtype) are optional (null to skip). */
int b200_mamba2_mixer_prefill(int dtype, const b200_mamba2_config* cfg, const b200_mamba2_weights* w,
	const void* u, void* out, int64_t batch, int64_t seqlen,
	const float* initial_states, void* conv_state_out, float* ssm_state_out,
	void* workspace, size_t workspace_bytes, void* stream);
/* Same call for callers holding HOST tensors (anyGPU's Tensor<dtype,CPU>::copy_to_cuda / copy_to_host pattern,
 * srcs/core/tensor.hpp:318-370): copies u_host in, runs the mixer, copies out_host back. The call is asynchronous and
 * ordered on `stream` (work queued on `stream` afterwards, or a synchronisation of it, sees out_host complete); inside,
 * the sequences of the batch are pipelined over three library-owned streams (copy-in, mixer, copy-out) so that the copy-in
 * of sequence i+1, the mixer of sequence i and the copy-out of sequence i-1 overlap. Pinned host memory is needed for that overlap.
 * The workspace must be b200_mamba2_mixer_prefill_host_workspace_bytes large (it also holds the staging tensors). */
size_t b200_mamba2_mixer_prefill_host_workspace_bytes(const b200_mamba2_config* cfg, int dtype, int64_t batch, int64_t seqlen);
int b200_mamba2_mixer_prefill_host(int dtype, const b200_mamba2_config* cfg, const b200_mamba2_weights* w,
	const void* u_host, void* out_host, int64_t batch, int64_t seqlen,
	void* workspace, size_t workspace_bytes, void* stream);
/* The same with flags. B200_HOST_OVERLAP: the caller vouches that this call needs nothing that was queued on `stream`
 * since the previous call of this function: u_host was filled by the CPU (not by work still queued on `stream`), the
 * weights have not been touched and nothing else has used the workspace in between. When the call then repeats the one before it (same workspace, stream, batch and sequence
 * length) it does not wait for that call to finish: its copy-in of slice i only waits until the earlier call's mixer
 * has read staging slice i, its mixer of slice i until the earlier copy-out of slice i is done (a slice is one sequence by
 * default; with the flag it is as many whole sequences as make ~4096 tokens, at least two slices per call, since a loop is
 * after throughput and a lone short sequence underfills the GPU). The copy-in of call k+1
 * so runs under the compute and the copy-out of call k, and a loop of calls is bound by the slower of one PCIe direction
 * and the compute instead of their sum per call. Ordering of out_host is unchanged (complete for work queued on `stream`
 * afterwards, and for a synchronisation of it). The mixer kernels of this entry point run on a library-owned stream. A
 * workspace is used from one stream at a time. During stream capture the flag is ignored. Other flag bits:
 * B200_ERR_UNSUPPORTED. */
enum { B200_HOST_OVERLAP = 1 };
int b200_mamba2_mixer_prefill_host_ex(int dtype, const b200_mamba2_config* cfg, const b200_mamba2_weights* w,
	const void* u_host, void* out_host, int64_t batch, int64_t seqlen,
	void* workspace, size_t workspace_bytes, void* stream, int flags);

/* ---- head-sharded tensor parallelism (prefill) -----------------------------------------------------------------
 * No counterpart in anyGPU (single device only, srcs/core/core.cpp:115-122). Rank r of TP owns nheads/TP heads: cfg_local
 * carries the LOCAL sizes (d_inner/TP, nheads/TP, the groups those heads use) and w the matching slices: in_proj columns
 * z_r | x_r | B,C of the rank's group(s) | dt_r (the row stride of that weight and of the local in_proj output is
 * d_in_proj_local rounded up to a multiple of 8, extra columns zero), conv / dt_bias / A_log / D / norm slices, out_proj rows.
 * _partial runs everything up to out_proj on the local heads and returns partial_out [T, d_model] (the rank's addend of
 * the un-normalised output) and sumsq [T] (its part of sum_j (y*silu(z))_j^2). The caller all-reduces both (sum) and calls
 * _finish, which scales row t by rsqrt(sumsq[t] / d_inner_global + eps): exactly the whole-row gated RMSNorm of the
 * unsharded layer, because the normalisation factor is a per-token scalar and commutes with out_proj. */
size_t b200_mamba2_mixer_prefill_tp_workspace_bytes(const b200_mamba2_config* cfg_local, int dtype, int64_t batch, int64_t seqlen);
int b200_mamba2_mixer_prefill_tp_partial(int dtype, const b200_mamba2_config* cfg_local, const b200_mamba2_weights* w,
	const void* u, void* partial_out, float* sumsq, int64_t batch, int64_t seqlen, void* conv_state_out, float* ssm_state_out,
	void* workspace, size_t workspace_bytes, void* stream);
int b200_mamba2_mixer_tp_finish(int dtype, void* out, const float* sumsq, int64_t rows, int64_t d_model, int64_t d_inner_global,
	float eps, void* stream);

size_t b200_mamba2_mixer_decode_workspace_bytes(const b200_mamba2_config* cfg, int dtype, int64_t batch);
/* One token per sequence: u_t [batch, d_model] -> out_t [batch, d_model]; conv_state [b, conv_dim, d_conv-1] (dtype) and
 * ssm_state [b,H,P,N] fp32 are advanced in place. */
int b200_mamba2_mixer_decode(int dtype, const b200_mamba2_config* cfg, const b200_mamba2_weights* w,
	const void* u_t, void* out_t, void* conv_state, float* ssm_state, int64_t batch,
	void* workspace, size_t workspace_bytes, void* stream);

/* ---- prefill continuation (chunked prefill) -----------------------------------------------------------------
 * `seqlen` more tokens for `batch` sequences whose state after the tokens seen so far is in conv_state [b, conv_dim, d_conv-1]
 * (dtype) and ssm_state [b,H,P,N] fp32 (zeros for a fresh sequence); both are advanced in place. A long prompt fed in pieces of
 * any length gives the same states and outputs as one call over the whole prompt (initial_states of
 * mamba_chunk_scan_combined_ref, scripts/zamba2/mamba_chunk_scan_comb.py:93-95,196-197, plus the conv1d history), and a decode
 * step may follow any piece. No counterpart in anyGPU. */
size_t b200_mamba2_mixer_prefill_continue_workspace_bytes(const b200_mamba2_config* cfg, int dtype, int64_t batch, int64_t seqlen);
int b200_mamba2_mixer_prefill_continue(int dtype, const b200_mamba2_config* cfg, const b200_mamba2_weights* w,
	const void* u, void* out, int64_t batch, int64_t seqlen, void* conv_state, float* ssm_state,
	void* workspace, size_t workspace_bytes, void* stream);

/* ---- packed variable-length batches ---------------------------------------------------------------------------
 * `nseq` sequences of different lengths stored back to back on the token axis: rows cu_seqlens[s] .. cu_seqlens[s+1]-1 of u and
 * out [total_tokens, d_model] belong to sequence s. cu_seqlens is a HOST array of nseq+1 non-decreasing offsets that starts at 0
 * (the `cu_seqlens` convention that scripts/zamba2/mamba_chunk_scan_comb.py:164-166 leaves unsupported). initial_states
 * [nseq,H,P,N] fp32 or NULL; conv_state_out [nseq, conv_dim, d_conv-1] (dtype) and ssm_state_out [nseq,H,P,N] fp32 or NULL. Every
 * sequence gets what b200_mamba2_mixer_prefill gives for it alone (bit for bit with chunk = 128, where both restart the cumulative
 * sums of dt*A at the same tokens; otherwise up to the rounding of those sums); an empty sequence hands on its initial state.
 * f16 batches with headdim = d_state = 64 take a fixed number of launches whatever the number of sequences (both projections and
 * the gated norm over all tokens; the conv1d and the dt stage of all sequences in one launch; the scan in one launch over
 * (sequence, head) pairs): many short sequences cost what one long one of the same token count costs. Other shapes and fp32 run
 * the conv1d and the scan sequence by sequence. The fixed-launch form copies its index arrays from pageable host memory to the
 * device inside the call (stream-ordered; the host arrays may be freed when the call returns), so the call cannot be captured
 * into a CUDA graph; cu_seqlens is read on the host during the call only. */
size_t b200_mamba2_mixer_prefill_varlen_workspace_bytes(const b200_mamba2_config* cfg, int dtype, int64_t total_tokens);
int b200_mamba2_mixer_prefill_varlen(int dtype, const b200_mamba2_config* cfg, const b200_mamba2_weights* w,
	const void* u, void* out, const int64_t* cu_seqlens, int64_t nseq,
	const float* initial_states, void* conv_state_out, float* ssm_state_out,
	void* workspace, size_t workspace_bytes, void* stream);

/* ---- sequence-parallel prefill: a long sequence split into consecutive segments, one per GPU ---------------------
 * No counterpart in anyGPU. The caller owns the communication; per segment (rank) r of R:
 *   1. _sp_begin(u_seg, u_halo = the d_conv-1 tokens before the segment, NULL for r = 0)   -> seg_state [b,H,P,N] fp32: the state the
 *      segment hands on for a ZERO incoming state; seg_logdecay [b,H] fp32: log of the factor by which it decays an incoming state
 *   2. all-gather seg_state and seg_logdecay over the ranks (two small tensors)
 *   3. b200_ssm_segment_prefix(gathered, nseg = r) -> state_in [b,H,P,N]: h <- exp(logdecay_q) h + seg_state_q for q < r
 *   4. _sp_finish(state_in)  -> out_seg [b, seglen, d_model]; ssm_state_out (optional) is the true state after the segment
 * The workspace of _sp_begin must reach _sp_finish unchanged. Segment lengths are free (they need not be multiples of the
 * chunk). The concatenated out_seg equal b200_mamba2_mixer_prefill over the whole sequence. */
size_t b200_mamba2_mixer_prefill_sp_workspace_bytes(const b200_mamba2_config* cfg, int dtype, int64_t batch, int64_t seglen);
int b200_mamba2_mixer_prefill_sp_begin(int dtype, const b200_mamba2_config* cfg, const b200_mamba2_weights* w,
	const void* u_seg, const void* u_halo, int64_t batch, int64_t seglen, float* seg_state, float* seg_logdecay, void* conv_state_out,
	void* workspace, size_t workspace_bytes, void* stream);
int b200_ssm_segment_prefix(const float* seg_states, const float* seg_logdecay, int nseg, int64_t batch, int64_t H, int64_t P,
	int64_t N, float* state_in, void* stream);
int b200_mamba2_mixer_prefill_sp_finish(int dtype, const b200_mamba2_config* cfg, const b200_mamba2_weights* w, void* out_seg,
	int64_t batch, int64_t seglen, const float* state_in, float* ssm_state_out, void* workspace, size_t workspace_bytes, void* stream);

/* ---- Zamba2 Mamba decoder layer: the mixer with its input norm and residual -----------------------------------
 * out = hidden + mixer(rms_norm(hidden, input_norm_weight, rms_eps)). No counterpart in anyGPU yet; the structure (input
 * RMSNorm, block, residual stream) is that of its hybrid block's other half, tensor_zamba_attention_decoder
 * (srcs/models/zamba2/zamba_attn_decoder.hpp:68-118). The residual is added in the epilogue of out_proj (f16) before the
 * single rounding of the result; `out` may alias `hidden`. Arguments as for the mixer entry points; the workspace holds the
 * normalised hidden states followed by the mixer's workspace. */
size_t b200_mamba2_decoder_prefill_workspace_bytes(const b200_mamba2_config* cfg, int dtype, int64_t batch, int64_t seqlen);
int b200_mamba2_decoder_prefill(int dtype, const b200_mamba2_config* cfg, const b200_mamba2_weights* w,
	const void* input_norm_weight, float rms_eps, const void* hidden, void* out, int64_t batch, int64_t seqlen,
	const float* initial_states, void* conv_state_out, float* ssm_state_out, void* workspace, size_t workspace_bytes, void* stream);
size_t b200_mamba2_decoder_decode_workspace_bytes(const b200_mamba2_config* cfg, int dtype, int64_t batch);
int b200_mamba2_decoder_decode(int dtype, const b200_mamba2_config* cfg, const b200_mamba2_weights* w,
	const void* input_norm_weight, float rms_eps, const void* hidden_t, void* out_t, void* conv_state, float* ssm_state, int64_t batch,
	void* workspace, size_t workspace_bytes, void* stream);

/* ---- per-stage timing of b200_mamba2_mixer_prefill -----------------------------------------------------------
 * No counterpart in anyGPU (its workflow is an external Nsight Compute CSV, scripts/perf_reports/plot_gemma_decoder.py:23-26).
 * When enabled, the prefill mixer records CUDA events on the caller's stream between its five stages
 * (in_proj, conv1d, ssd, gated_rmsnorm, out_proj) for up to 256 calls. b200_stage_timing_collect waits for the recorded
 * calls, writes the SUM of each stage's milliseconds over those calls to stage_ms[5] and their number to *calls, and
 * starts a new window. enable = 2 records only the two events around in_proj, and only in every fourth call (the other
 * entries of stage_ms stay 0, *calls counts the recorded calls): an event between two kernels costs about 2.5 us of the
 * step, so a harness that times whole steps and wants the dominant kernel's duration from the same steps uses 2 there and
 * 1 in a pass of its own. Calls captured into a CUDA graph while timing is enabled record their events on every replay
 * (collect after the replay, not after the capture; a window then holds the calls of one capture). Not thread safe;
 * meant for a benchmark harness. */
int b200_stage_timing_enable(int enable);
int b200_stage_timing_collect(float* stage_ms, int* calls);

#ifdef __cplusplus
}
#endif
#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
#endif /* B200_MAMBA2_H */
