// CPU oracle for the Mamba2 mixer forward path of anyGPU's Zamba2 blocks.
//
// THIS FILE IS TEST INFRASTRUCTURE. It is the checker that the CUDA path is compared
// against and the CPU baseline that the benchmark times. Nothing in the shipped library
// or its host layer links, loads or calls it.
//
// Every function is a plain-loop fp32 restatement of the reference algorithm it cites
// (paths are relative to the anyGPU project root). Where the reference has C++ CPU code
// (linear, causal conv1d, silu/mul/rms_norm) the restatement keeps its loop order and
// accumulation type, so results agree bit-for-bit with the reference compiled from its own
// sources (checked by the tests when that build is present). Where the reference has only
// its PyTorch script (the SSD chunked scan) the restatement follows the script's stages and
// is pinned by golden vectors generated from that script.
//
// Parallelism: host threads over independent rows / (batch, head) pairs only (single thread
// unless orc_set_num_threads is called); the arithmetic order inside one output element never
// depends on the thread count.

#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>
#include <algorithm>

#include <thread>
#include <atomic>
#include <functional>

namespace {

int g_threads = 1;

// Runs body(i) for i in [0, n) on g_threads host threads (dynamic distribution of indices).
template <class F>
void pfor(int64_t n, F body)
{
	const int nt = static_cast<int>(std::min<int64_t>(g_threads, n));
	if (nt <= 1)
	{
		for (int64_t i = 0; i < n; ++i) body(i);
		return;
	}
	std::atomic<int64_t> next(0);
	std::vector<std::thread> pool;
	for (int t = 0; t < nt; ++t)
	{
		pool.emplace_back([&]() {
			for (;;)
			{
				const int64_t i = next.fetch_add(1);
				if (i >= n) return;
				body(i);
			}
		});
	}
	for (auto& th : pool) th.join();
}

// Round-to-nearest-even through IEEE binary16, as the device does when an op writes an
// f16 tensor. Used only by the *_f16io entry points below.
inline float round_f16(float v)
{
	return static_cast<float>(static_cast<_Float16>(v));
}

// torch.nn.functional.softplus with beta=1, threshold=20
// (scripts/zamba2/mamba_chunk_scan_comb.py:45 calls F.softplus).
inline float softplus_f(float v)
{
	return v > 20.f ? v : log1pf(expf(v));
}

// srcs/ops/math_ops.hpp:31 and srcs/fused/causal_conv1d.hpp:79 : x / ((dtype)1.0 + exp(-x)).
// With the host compiler the unqualified exp(float) call binds to the C library's double
// exp(double), so the quotient is formed in double and rounded to float on assignment.
inline float ref_silu(float v)
{
	return static_cast<float>(static_cast<double>(v) / (static_cast<double>(1.0f) + std::exp(static_cast<double>(-v))));
}

}  // namespace

extern "C" {

int orc_num_threads()
{
	return g_threads;
}

// n <= 0 selects every hardware thread of the host.
void orc_set_num_threads(int n)
{
	if (n <= 0) n = static_cast<int>(std::thread::hardware_concurrency());
	g_threads = n < 1 ? 1 : n;
}

void orc_round_f16(const float* x, float* y, int64_t n)
{
	for (int64_t i = 0; i < n; ++i) y[i] = round_f16(x[i]);
}

// Y[M,N] = X[M,K] . W[K,N]; fp32, sequential accumulation over k.
// Follows tensor_mm<CPU> (srcs/ops/mm_ops.hpp:11-45) as used by tensor_linear without bias
// (srcs/ops/mm_ops.hpp:206-232). W is (in_features, out_features) row-major.
void orc_linear_f32(const float* x, const float* w, float* y, int64_t M, int64_t K, int64_t N)
{
	pfor(M, [&](int64_t r)
	{
		for (int64_t c = 0; c < N; ++c)
		{
			float acc = 0.f;
			for (int64_t l = 0; l < K; ++l)
			{
				acc += x[r * K + l] * w[l * N + c];
			}
			y[r * N + c] = acc;
		}
	});
}

// Same result as orc_linear_f32 (identical per-element accumulation order), but with the
// k loop outermost inside a row so W is streamed by rows. Used for the larger parity cases.
void orc_linear_f32_fast(const float* x, const float* w, float* y, int64_t M, int64_t K, int64_t N)
{
	pfor(M, [&](int64_t r)
	{
		float* yr = y + r * N;
		for (int64_t c = 0; c < N; ++c) yr[c] = 0.f;
		for (int64_t l = 0; l < K; ++l)
		{
			const float xv = x[r * K + l];
			const float* wr = w + l * N;
			for (int64_t c = 0; c < N; ++c)
			{
				yr[c] += xv * wr[c];
			}
		}
	});
}

// y[b,d,s] = silu(bias[d] + sum_k w[d,k] * x[b,d,s+k-(W-1)]), zero left padding.
// Follows tensor_causal_conv1d<CPU> (srcs/fused/causal_conv1d.hpp:24-87): accumulator starts
// at 0, taps added for k = 0..W-1, bias added last, then out / (1 + exp(-out)).
void orc_causal_conv1d_f32(const float* x, const float* w, const float* bias, float* y,
	int64_t B, int64_t D, int64_t S, int64_t W)
{
	pfor(B * D, [&](int64_t row)
	{
		const int64_t dix = row % D;
		const float* xr = x + row * S;
		float* yr = y + row * S;
		const float* wr = w + dix * W;
		for (int64_t six = 0; six < S; ++six)
		{
			float out = 0.f;
			for (int64_t k = 0; k < W; ++k)
			{
				const int64_t delta = k + 1 + six - W;
				if (delta >= 0) out += wr[k] * xr[delta];
			}
			out += bias[dix];
			out = ref_silu(out);
			yr[six] = out;
		}
	});
}

// One decode step of the causal conv1d: conv_state[b,d,W-1] holds the previous W-1 inputs
// (oldest first). Output equals column t of orc_causal_conv1d_f32 run on the concatenated
// history (same tap order: oldest input times w[d,0] first). The state is then advanced.
// The reference has no decode path; this restates srcs/fused/causal_conv1d.hpp:60-81 for a
// single column.
void orc_causal_conv1d_update_f32(const float* x_t, float* conv_state, const float* w, const float* bias,
	float* y_t, int64_t B, int64_t D, int64_t W)
{
	const int64_t SW = W - 1;
	pfor(B * D, [&](int64_t row)
	{
		const int64_t dix = row % D;
		float* st = conv_state + row * SW;
		const float* wr = w + dix * W;
		float out = 0.f;
		for (int64_t k = 0; k < SW; ++k) out += wr[k] * st[k];
		out += wr[SW] * x_t[row];
		out += bias[dix];
		out = ref_silu(out);
		y_t[row] = out;
		for (int64_t k = 0; k + 1 < SW; ++k) st[k] = st[k + 1];
		if (SW > 0) st[SW - 1] = x_t[row];
	});
}

// y = x / sqrt(mean_row(x^2) + eps) * (w + delta): tensor_rms_norm<CPU> over the last axis (srcs/ops/norm_ops.hpp:134-191),
// delta = 1 for its zero_centered flag. Sequential fp32 sum of squares; the unqualified sqrt(float) at :188 is the double
// overload on the host, so the quotient and the product with w are formed in double and rounded once.
void orc_rms_norm_f32(const float* x, const float* w, float* y, int64_t rows, int64_t d, float eps, int zero_centered)
{
	const float delta = zero_centered ? 1.f : 0.f;
	pfor(rows, [&](int64_t r)
	{
		float acc = 0.f;
		for (int64_t i = 0; i < d; ++i) acc += x[r * d + i] * x[r * d + i];
		const float ms = acc / static_cast<float>(d);
		for (int64_t i = 0; i < d; ++i)
			y[r * d + i] = static_cast<float>((static_cast<double>(x[r * d + i]) / std::sqrt(static_cast<double>(ms + eps)))
				* static_cast<double>(w[i] + delta));
	});
}

// y = rms_norm(x * silu(z)) * w over groups of `gsize` elements of the last axis.
// Follows tensor_zamba_gated_rmsnorm (srcs/models/zamba2/zamba_gated_rmsnorm.hpp:9-23):
// tensor_silu (srcs/ops/math_ops.hpp:16-35), tensor_mul (srcs/ops/binary_ops.hpp:103-121),
// tensor_rms_norm<CPU> (srcs/ops/norm_ops.hpp:134-194): sequential fp32 sum of squares,
// mean, then (x / sqrt(mean + eps)) * w. The reference ignores its gsize argument and
// normalises the whole row; pass gsize == d for that behaviour.
void orc_gated_rmsnorm_f32(const float* x, const float* z, const float* w, float* y,
	int64_t rows, int64_t d, int64_t gsize, float eps)
{
	const int64_t ngroups = d / gsize;
	pfor(rows, [&](int64_t r)
	{
		std::vector<float> gated(gsize);
		for (int64_t g = 0; g < ngroups; ++g)
		{
			const int64_t base = r * d + g * gsize;
			float acc = 0.f;
			for (int64_t i = 0; i < gsize; ++i)
			{
				const float zv = z[base + i];
				const float s = ref_silu(zv);
				const float gv = x[base + i] * s;
				gated[i] = gv;
				acc += gv * gv;
			}
			const float ms = acc / static_cast<float>(gsize);
			for (int64_t i = 0; i < gsize; ++i)
			{
				// unqualified sqrt(float) in srcs/ops/norm_ops.hpp:188 is the double overload on the host
				y[base + i] = static_cast<float>((static_cast<double>(gated[i]) / std::sqrt(static_cast<double>(ms + eps)))
					* static_cast<double>(w[g * gsize + i]));
			}
		}
	});
}

// SSD chunked selective scan, fp32.
// Follows mamba_chunk_scan_combined_ref (scripts/zamba2/mamba_chunk_scan_comb.py:167-215):
//   chunk_cumsum_ref  :32-48   zero-pad dt to a chunk multiple BEFORE bias and softplus, dA = dt*A, in-chunk cumsum
//   chunk_state_ref   :51-80   states[b,c,h,p,n] = sum_l B[l,n] exp(dAcs[last]-dAcs[l]) dt[l] x[l,p]
//   state_passing_ref :83-106  prefix over chunks through exp(segment sums), initial state prepended
//   chunk_scan_ref    :109-160 (C.B^T o decay o causal mask).(dt x) + (C.prev^T) exp(dAcs) + D x
// x [b,l,H,P], dt [b,l,H], A [H], Bm/Cm [b,l,G,N], D [H] (may be null), dt_bias [H] (may be null),
// init_state [b,H,P,N] (may be null) -> y [b,l,H,P], final_state [b,H,P,N].
// All intermediates (decays, scores, chunk states) stay fp32; callers round whole-op outputs only.
void orc_ssd_chunk_scan_f32(const float* x, const float* dt_in, const float* A, const float* Bm, const float* Cm,
	const float* D, const float* dt_bias, const float* init_state, float* y, float* final_state,
	int64_t batch, int64_t seqlen, int64_t H, int64_t P, int64_t G, int64_t N, int64_t Q, int dt_softplus)
{
	const int64_t nchunks = (seqlen + Q - 1) / Q;
	const int64_t hpg = H / G;
	pfor(batch * H, [&](int64_t bh)
	{
		{
			const int64_t b = bh / H, h = bh % H;
			const int64_t g = h / hpg;
			std::vector<float> dt(nchunks * Q), dacs(nchunks * Q);
			// chunk_cumsum_ref
			for (int64_t c = 0; c < nchunks; ++c)
			{
				float run = 0.f;
				for (int64_t l = 0; l < Q; ++l)
				{
					const int64_t t = c * Q + l;
					float v = t < seqlen ? dt_in[(b * seqlen + t) * H + h] : 0.f;
					if (dt_bias) v += dt_bias[h];
					if (dt_softplus) v = softplus_f(v);
					dt[t] = v;
					run += v * A[h];
					dacs[t] = run;
				}
			}
			// chunk_state_ref
			std::vector<float> states(nchunks * P * N, 0.f);
			for (int64_t c = 0; c < nchunks; ++c)
			{
				const float last = dacs[c * Q + Q - 1];
				float* st = states.data() + c * P * N;
				for (int64_t l = 0; l < Q; ++l)
				{
					const int64_t t = c * Q + l;
					if (t >= seqlen) break;  // padded x and B are zero
					const float sc = expf(last - dacs[t]) * dt[t];
					const float* xr = x + ((b * seqlen + t) * H + h) * P;
					const float* br = Bm + ((b * seqlen + t) * G + g) * N;
					for (int64_t p = 0; p < P; ++p)
					{
						const float xv = xr[p] * sc;
						for (int64_t n = 0; n < N; ++n) st[p * N + n] += br[n] * xv;
					}
				}
			}
			// state_passing_ref: cs = cumsum([0, dA_last[0..nchunks-1]]); out[z] = sum_{c<=z} exp(cs[z]-cs[c]) cat[c]
			std::vector<float> cs(nchunks + 1);
			cs[0] = 0.f;
			for (int64_t c = 0; c < nchunks; ++c) cs[c + 1] = cs[c] + dacs[c * Q + Q - 1];
			std::vector<float> prev((nchunks + 1) * P * N, 0.f);
			for (int64_t z = 0; z <= nchunks; ++z)
			{
				float* out = prev.data() + z * P * N;
				for (int64_t c = 0; c <= z; ++c)
				{
					const float dec = expf(cs[z] - cs[c]);
					const float* src = nullptr;
					if (c == 0)
					{
						if (!init_state) continue;
						src = init_state + (b * H + h) * P * N;
					}
					else
					{
						src = states.data() + (c - 1) * P * N;
					}
					for (int64_t i = 0; i < P * N; ++i) out[i] += dec * src[i];
				}
			}
			if (final_state)
			{
				std::memcpy(final_state + (b * H + h) * P * N, prev.data() + nchunks * P * N, sizeof(float) * P * N);
			}
			// chunk_scan_ref
			std::vector<float> score(Q);
			for (int64_t c = 0; c < nchunks; ++c)
			{
				const float* pst = prev.data() + c * P * N;
				for (int64_t l = 0; l < Q; ++l)
				{
					const int64_t t = c * Q + l;
					if (t >= seqlen) break;
					const float* cr = Cm + ((b * seqlen + t) * G + g) * N;
					float* yr = y + ((b * seqlen + t) * H + h) * P;
					for (int64_t s = 0; s <= l; ++s)
					{
						const int64_t ts = c * Q + s;
						const float* br = Bm + ((b * seqlen + ts) * G + g) * N;
						float cb = 0.f;
						for (int64_t n = 0; n < N; ++n) cb += cr[n] * br[n];
						score[s] = cb * expf(dacs[t] - dacs[ts]) * dt[ts];
					}
					const float dec_out = expf(dacs[t]);
					const float* xt = x + ((b * seqlen + t) * H + h) * P;
					for (int64_t p = 0; p < P; ++p)
					{
						float acc = 0.f;
						for (int64_t s = 0; s <= l; ++s)
						{
							acc += score[s] * x[((b * seqlen + c * Q + s) * H + h) * P + p];
						}
						float accp = 0.f;
						for (int64_t n = 0; n < N; ++n) accp += cr[n] * pst[p * N + n];
						float out = acc + accp * dec_out;
						if (D) out += xt[p] * D[h];
						yr[p] = out;
					}
				}
			}
		}
	});
}

// Per-token selective-state recurrence over a whole sequence, fp32. Independent second
// statement of the same mathematics (no chunking): h <- exp(dt A) h + dt x (x) B ; y = h.C + D x.
// This is what the decode step computes; it is mathematically identical to
// mamba_chunk_scan_combined_ref (scripts/zamba2/mamba_chunk_scan_comb.py:167-215) when
// seqlen is a multiple of the chunk size. state [b,H,P,N] is read as the initial state and
// overwritten with the final one.
void orc_ssd_recurrence_f32(const float* x, const float* dt_in, const float* A, const float* Bm, const float* Cm,
	const float* D, const float* dt_bias, float* state, float* y,
	int64_t batch, int64_t seqlen, int64_t H, int64_t P, int64_t G, int64_t N, int dt_softplus)
{
	const int64_t hpg = H / G;
	pfor(batch * H, [&](int64_t bh)
	{
		{
			const int64_t b = bh / H, h = bh % H;
			const int64_t g = h / hpg;
			float* st = state + (b * H + h) * P * N;
			for (int64_t t = 0; t < seqlen; ++t)
			{
				float dtv = dt_in[(b * seqlen + t) * H + h];
				if (dt_bias) dtv += dt_bias[h];
				if (dt_softplus) dtv = softplus_f(dtv);
				const float dA = expf(dtv * A[h]);
				const float* xr = x + ((b * seqlen + t) * H + h) * P;
				const float* br = Bm + ((b * seqlen + t) * G + g) * N;
				const float* cr = Cm + ((b * seqlen + t) * G + g) * N;
				float* yr = y + ((b * seqlen + t) * H + h) * P;
				for (int64_t p = 0; p < P; ++p)
				{
					const float dx = dtv * xr[p];
					float acc = 0.f;
					for (int64_t n = 0; n < N; ++n)
					{
						const float s = st[p * N + n] * dA + dx * br[n];
						st[p * N + n] = s;
						acc += s * cr[n];
					}
					if (D) acc += D[h] * xr[p];
					yr[p] = acc;
				}
			}
		}
	});
}

// ---------------------------------------------------------------------------------------
// Mixer composition (prefill). Dataflow of a Zamba2 Mamba2 layer assembled from the ops above:
//   zxbcdt = linear(u, W_in)                       [T, 2*d_inner + 2*G*N + H]  split z | xBC | dt
//   xBC    = causal_conv1d(xBC^T)^T                split x[d_inner] | B[G*N] | C[G*N]
//   y      = ssd(x, dt, A = -exp(A_log), B, C, D, dt_bias, softplus)
//   g      = gated_rmsnorm(y, z, norm_w, eps)
//   out    = linear(g, W_out)
// f16io != 0 rounds every op OUTPUT tensor (zxbcdt, conv out, y, g, out) to binary16, which is
// what a chain of Tensor<float16> ops does; arithmetic inside each op stays fp32.
// Optional outputs (may be null): zxbcdt_out [T,d_in_proj], xbc_out [T,conv_dim] (after conv),
// y_out [T,d_inner], g_out [T,d_inner], final_state [b,H,P,N], conv_state_out [b,conv_dim,W-1]
// (last W-1 pre-conv xBC columns, oldest first; zero where the sequence is shorter).
void orc_mamba2_mixer_prefill_f32(const float* u, const float* W_in, const float* conv_w, const float* conv_b,
	const float* dt_bias, const float* A_log, const float* D, const float* norm_w, const float* W_out,
	const float* init_state,
	float* out, float* zxbcdt_out, float* xbc_out, float* y_out, float* g_out, float* final_state, float* conv_state_out,
	int64_t batch, int64_t seqlen, int64_t d_model, int64_t d_inner, int64_t H, int64_t P, int64_t G, int64_t N,
	int64_t W, int64_t Q, int64_t norm_gsize, float eps, int f16io)
{
	const int64_t T = batch * seqlen;
	const int64_t conv_dim = d_inner + 2 * G * N;
	const int64_t d_in_proj = 2 * d_inner + 2 * G * N + H;
	std::vector<float> zx(T * d_in_proj);
	orc_linear_f32_fast(u, W_in, zx.data(), T, d_model, d_in_proj);
	if (f16io) orc_round_f16(zx.data(), zx.data(), T * d_in_proj);
	if (zxbcdt_out) std::memcpy(zxbcdt_out, zx.data(), sizeof(float) * T * d_in_proj);

	// (b, c, l) layout for the conv, as the reference op expects
	std::vector<float> xin(batch * conv_dim * seqlen), xconv(batch * conv_dim * seqlen);
	for (int64_t b = 0; b < batch; ++b)
		for (int64_t l = 0; l < seqlen; ++l)
			for (int64_t c = 0; c < conv_dim; ++c)
				xin[(b * conv_dim + c) * seqlen + l] = zx[(b * seqlen + l) * d_in_proj + d_inner + c];
	if (conv_state_out)
	{
		for (int64_t b = 0; b < batch; ++b)
			for (int64_t c = 0; c < conv_dim; ++c)
				for (int64_t k = 0; k < W - 1; ++k)
				{
					const int64_t l = seqlen - (W - 1) + k;
					conv_state_out[(b * conv_dim + c) * (W - 1) + k] = l >= 0 ? xin[(b * conv_dim + c) * seqlen + l] : 0.f;
				}
	}
	orc_causal_conv1d_f32(xin.data(), conv_w, conv_b, xconv.data(), batch, conv_dim, seqlen, W);
	if (f16io) orc_round_f16(xconv.data(), xconv.data(), batch * conv_dim * seqlen);

	std::vector<float> xs(T * d_inner), Bs(T * G * N), Cs(T * G * N), dts(T * H), Av(H);
	for (int64_t b = 0; b < batch; ++b)
		for (int64_t l = 0; l < seqlen; ++l)
		{
			const int64_t t = b * seqlen + l;
			for (int64_t c = 0; c < conv_dim; ++c)
			{
				const float v = xconv[(b * conv_dim + c) * seqlen + l];
				if (xbc_out) xbc_out[t * conv_dim + c] = v;
				if (c < d_inner) xs[t * d_inner + c] = v;
				else if (c < d_inner + G * N) Bs[t * G * N + (c - d_inner)] = v;
				else Cs[t * G * N + (c - d_inner - G * N)] = v;
			}
			for (int64_t h = 0; h < H; ++h) dts[t * H + h] = zx[t * d_in_proj + d_inner + conv_dim + h];
		}
	for (int64_t h = 0; h < H; ++h) Av[h] = -expf(A_log[h]);

	std::vector<float> y(T * d_inner);
	orc_ssd_chunk_scan_f32(xs.data(), dts.data(), Av.data(), Bs.data(), Cs.data(), D, dt_bias, init_state,
		y.data(), final_state, batch, seqlen, H, P, G, N, Q, 1);
	if (f16io) orc_round_f16(y.data(), y.data(), T * d_inner);
	if (y_out) std::memcpy(y_out, y.data(), sizeof(float) * T * d_inner);

	std::vector<float> zs(T * d_inner), gn(T * d_inner);
	for (int64_t t = 0; t < T; ++t)
		std::memcpy(zs.data() + t * d_inner, zx.data() + t * d_in_proj, sizeof(float) * d_inner);
	orc_gated_rmsnorm_f32(y.data(), zs.data(), norm_w, gn.data(), T, d_inner, norm_gsize, eps);
	if (f16io) orc_round_f16(gn.data(), gn.data(), T * d_inner);
	if (g_out) std::memcpy(g_out, gn.data(), sizeof(float) * T * d_inner);

	orc_linear_f32_fast(gn.data(), W_out, out, T, d_inner, d_model);
	if (f16io) orc_round_f16(out, out, T * d_model);
}

// One decode step of the mixer for `batch` sequences (one token each). conv_state
// [b,conv_dim,W-1] and ssm_state [b,H,P,N] are advanced in place. Same rounding rule as above.
void orc_mamba2_mixer_decode_f32(const float* u, const float* W_in, const float* conv_w, const float* conv_b,
	const float* dt_bias, const float* A_log, const float* D, const float* norm_w, const float* W_out,
	float* conv_state, float* ssm_state, float* out,
	int64_t batch, int64_t d_model, int64_t d_inner, int64_t H, int64_t P, int64_t G, int64_t N,
	int64_t W, int64_t norm_gsize, float eps, int f16io)
{
	const int64_t conv_dim = d_inner + 2 * G * N;
	const int64_t d_in_proj = 2 * d_inner + 2 * G * N + H;
	std::vector<float> zx(batch * d_in_proj);
	orc_linear_f32_fast(u, W_in, zx.data(), batch, d_model, d_in_proj);
	if (f16io) orc_round_f16(zx.data(), zx.data(), batch * d_in_proj);

	std::vector<float> xt(batch * conv_dim), xc(batch * conv_dim);
	for (int64_t b = 0; b < batch; ++b)
		std::memcpy(xt.data() + b * conv_dim, zx.data() + b * d_in_proj + d_inner, sizeof(float) * conv_dim);
	orc_causal_conv1d_update_f32(xt.data(), conv_state, conv_w, conv_b, xc.data(), batch, conv_dim, W);
	if (f16io) orc_round_f16(xc.data(), xc.data(), batch * conv_dim);

	std::vector<float> xs(batch * d_inner), Bs(batch * G * N), Cs(batch * G * N), dts(batch * H), Av(H), y(batch * d_inner);
	for (int64_t b = 0; b < batch; ++b)
	{
		std::memcpy(xs.data() + b * d_inner, xc.data() + b * conv_dim, sizeof(float) * d_inner);
		std::memcpy(Bs.data() + b * G * N, xc.data() + b * conv_dim + d_inner, sizeof(float) * G * N);
		std::memcpy(Cs.data() + b * G * N, xc.data() + b * conv_dim + d_inner + G * N, sizeof(float) * G * N);
		std::memcpy(dts.data() + b * H, zx.data() + b * d_in_proj + d_inner + conv_dim, sizeof(float) * H);
	}
	for (int64_t h = 0; h < H; ++h) Av[h] = -expf(A_log[h]);
	orc_ssd_recurrence_f32(xs.data(), dts.data(), Av.data(), Bs.data(), Cs.data(), D, dt_bias, ssm_state, y.data(),
		batch, 1, H, P, G, N, 1);
	if (f16io) orc_round_f16(y.data(), y.data(), batch * d_inner);

	std::vector<float> zs(batch * d_inner), gn(batch * d_inner);
	for (int64_t b = 0; b < batch; ++b)
		std::memcpy(zs.data() + b * d_inner, zx.data() + b * d_in_proj, sizeof(float) * d_inner);
	orc_gated_rmsnorm_f32(y.data(), zs.data(), norm_w, gn.data(), batch, d_inner, norm_gsize, eps);
	if (f16io) orc_round_f16(gn.data(), gn.data(), batch * d_inner);
	orc_linear_f32_fast(gn.data(), W_out, out, batch, d_inner, d_model);
	if (f16io) orc_round_f16(out, out, batch * d_model);
}

}  // extern "C"
